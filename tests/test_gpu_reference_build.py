"""GPU test against the reference's OWN CUDA build (oracle/_ref/quantized_mf, compiled from the reference
sources by `make -C oracle ref`; the binary travels with the repository snapshot, the sources do not): the
statistical half of the parity criterion.  Both programs train the same seeded synthetic ratings - written
once as the TSV the reference reads - with the same hyper-parameters; Hogwild ordering makes the trajectories
nondeterministic, so what is compared is the final test RMSE.  The engine must not be worse than the reference
build by more than 0.5 % relative; it may be better, within 3 %: on these small sets the reference's 2048 racing
warps lose updates of popular rows that the engine keeps (user rows are written back as reductions), so after
the same number of epochs the engine is ahead by up to 1.5 %, and the gap closes as both converge (on the
100M-rating set the two builds end within 0.3 %).  Skipped when the binary is absent."""
import os
import re
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "quantized_mf")
BIN = os.path.join(ROOT, "icdm-2021_mascot_b200", "bin")
EPOCH_LINE = re.compile(r"(?:^|(?<= ))(\d+) ([0-9.]+(?:e-?\d+)?) ([0-9.]+(?:e-?\d+)?)$", re.M)


def final_rmse(cmd):
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-1500:]
    ep = EPOCH_LINE.findall(out.stdout)
    assert ep, out.stdout[-1500:]
    return float(ep[-1][2]), len(ep)


@pytest.mark.parametrize("name,version,k,extra", [
    ("c1", 5, 64, []),                                                                       # FP32 SGD
    ("c2_tenth", 1, 128, ["-ug", "30", "-ig", "30", "-s", "0.05", "-it", "2", "-e", "20"]),   # MASCOT, switching on
])
def test_final_rmse_not_worse_than_the_reference_build_by_half_a_percent(mascot, synth, tmp_path, name, version, k, extra):
    if not os.path.exists(REF):
        pytest.skip("the reference build is not present (make -C oracle ref)")
    cfg = synth.CONFIGS["c1"] if name == "c1" else synth.scaled(synth.CONFIGS["c2"], 0.1)
    train, test = synth.generate(cfg, seed=4)
    d = str(tmp_path)
    mascot.write_binary_ratings(f"{d}/train.bin", train, cfg["users"], cfg["items"])
    mascot.write_binary_ratings(f"{d}/test.bin", test, cfg["users"], cfg["items"])
    for part in ("train", "test"):
        subprocess.check_call([os.path.join(BIN, "convert_ratings"), f"{d}/{part}.bin", f"{d}/{part}.tsv", "tsv"])
    hy = cfg["hyper"]
    epochs = 20 if name == "c1" else 30
    common = ["-i", f"{d}/train.tsv", "-y", f"{d}/test.tsv", "-k", str(k), "-l", str(epochs), "-a", str(hy["learning_rate"]),
              "-d", str(hy["decay"]), "-b", str(hy["lam"]), "-v", str(version)] + extra
    ref, n_ref = final_rmse([REF] + common + ["-wg", "2048", "-bl", "128"])
    ours, n_ours = final_rmse([os.path.join(BIN, "quantized_mf")] + common)
    assert n_ref == n_ours == epochs
    assert np.isfinite(ref) and np.isfinite(ours)
    assert ours <= 1.005 * ref, f"final test RMSE {ours:.5f} is worse than the reference build's {ref:.5f} by more than 0.5 %"
    assert ours >= 0.97 * ref, f"final test RMSE {ours:.5f} is implausibly far below the reference build's {ref:.5f}"
