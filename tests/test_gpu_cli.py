"""GPU tests of the command-line tools: quantized_mf trains from rating files in the reference's
formats and writes a model that test_mf re-evaluates to the same RMSE."""
import os
import re
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "icdm-2021_mascot_b200", "bin")
# "<epoch> <lr> <rmse>" at the end of a line; like in the reference, the first one follows the group
# listing of the MASCOT variant on the same line (that listing ends without a newline)
EPOCH_LINE = re.compile(r"(?:^|(?<= ))(\d+) ([0-9.]+(?:e-?\d+)?) ([0-9.]+(?:e-?\d+)?)$", re.M)


def write_dataset(synth, d, name_train, name_test, item_first=False, seed=3):
    cfg = dict(users=600, items=300, n_train=40000, n_test=6000, k=64, version=5,
               user_deg=("zipf", 0.8), item_deg=("zipf", 0.8), grid="half0.5_5", hyper={})
    train, test = synth.generate(cfg, seed=seed)
    rng = np.random.default_rng(seed)
    uid = rng.permutation(5000)[:cfg["users"]] + 1          # sparse original ids with gaps
    iid = rng.permutation(3000)[:cfg["items"]] + 1
    for recs, name in ((train, name_train), (test, name_test)):
        with open(os.path.join(d, name), "w") as f:
            for r in recs:
                a, b = uid[r["u"]], iid[r["i"]]
                if item_first:
                    a, b = b, a
                f.write(f"{a}\t{b}\t{r['r']:g}\n")
    return train, test


def run(cmd):
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    return out.stdout


@pytest.mark.parametrize("version,k", [(5, 64), (4, 128), (7, 64), (2, 128), (3, 64), (6, 128), (8, 128)])
def test_train_save_and_reevaluate_original_id_models(synth, tmp_path, version, k):
    d = str(tmp_path)
    write_dataset(synth, d, "train.tsv", "test.tsv")
    out = run([os.path.join(BIN, "quantized_mf"), "-i", f"{d}/train.tsv", "-y", f"{d}/test.tsv", "-o", f"{d}/model",
               "-k", str(k), "-l", "12", "-a", "0.02", "-b", "0.05", "-v", str(version), "-wg", "64", "-seed", "5"])
    assert f"Latent features             : {k}" in out and "Num of workers              : 64" in out
    assert "The number of users         : 600" in out
    ep = EPOCH_LINE.findall(out)
    assert [int(e[0]) for e in ep] == list(range(1, 13))
    rm = [float(e[2]) for e in ep]
    assert rm[-1] < rm[0] and np.isfinite(rm).all()
    assert "Parameters update per epoch" in out and "Save trained model..." in out
    head = open(f"{d}/model.txt").readline().split()
    assert int(head[2]) == k and int(head[0]) <= 5001 and int(head[1]) <= 3001
    ev = run([os.path.join(BIN, "test_mf"), "-i", f"{d}/model.txt", "-y", f"{d}/test.tsv", "-v", str(version)])
    got = float(re.search(r"RMSE : ([0-9.eE+-]+)", ev).group(1))
    assert abs(got - rm[-1]) <= 2e-4 * rm[-1]      # the text model keeps 6 significant digits


def test_mascot_variant_with_reconst_outputs(synth, tmp_path):
    d = str(tmp_path / "ml25M_like")                      # "25M" in the path: item-first columns
    os.makedirs(d)
    write_dataset(synth, d, "train.tsv", "test.tsv", item_first=True)
    out = run([os.path.join(BIN, "quantized_mf"), "-i", f"{d}/train.tsv", "-y", f"{d}/test.tsv", "-o", f"{d}/m",
               "-k", "128", "-l", "10", "-a", "0.02", "-b", "0.015", "-v", "1", "-ug", "8", "-ig", "6", "-s", "0.1",
               "-it", "2", "-e", "0.5", "-rc", "1", "-wg", "64"])
    assert "The number of user groups   :" in out and "<User groups>" in out and "<Item groups>" in out
    ep = EPOCH_LINE.findall(out)
    assert len(ep) == 10
    assert out.count("<User groups>") == 2               # check epochs 5 and 7 (index), never the last
    head = open(f"{d}/m_reconst.txt").readline().split()
    assert head == ["600", "300", "128"]
    rec = open(f"{d}/reconst_test.tsv").read().split("\n")
    first = rec[0].split("\t")
    assert len(first) == 3 and int(first[0]) < 300 and int(first[1]) < 600      # item first, sorted-index ids
    ev = run([os.path.join(BIN, "test_mf"), "-i", f"{d}/m_reconst.txt", "-y", f"{d}/reconst_test.tsv", "-v", "1"])
    got = float(re.search(r"RMSE : ([0-9.eE+-]+)", ev).group(1))
    assert abs(got - float(ep[-1][2])) <= 2e-4 * got


def test_binary_input_binary_model_timing_block_and_no_test_file(synth, tmp_path):
    """Additive surface: binary rating files (mapped, compact ids), -ob 1 binary model read back by test_mf,
    the reference's full timing report, the chosen worker count as a number, and a run without -y."""
    d = str(tmp_path)
    train, test = write_dataset(synth, d, "train.tsv", "test.tsv")
    conv, qmf, tmf = (os.path.join(BIN, x) for x in ("convert_ratings", "quantized_mf", "test_mf"))
    run([conv, f"{d}/train.tsv", f"{d}/train.bin", "bin"])
    # the test file must share the id space: write it in the compact ids of the training conversion
    import importlib.util
    spec = importlib.util.spec_from_file_location("mascot_binding", os.path.join(ROOT, "icdm-2021_mascot_b200", "mascot.py"))
    M = importlib.util.module_from_spec(spec); spec.loader.exec_module(M)
    tr = np.fromfile(f"{d}/train.bin", M.RATING, offset=32)
    # first-seen compaction of the text file: rebuild the maps from the text and the binary side by side
    txt = np.loadtxt(f"{d}/train.tsv", dtype=np.int64, usecols=(0, 1))
    umap = dict(zip(txt[:, 0].tolist(), tr["u"].tolist())); imap = dict(zip(txt[:, 1].tolist(), tr["i"].tolist()))
    tt = np.loadtxt(f"{d}/test.tsv")
    keep = [(umap[int(a)], imap[int(b)], c) for a, b, c in tt if int(a) in umap and int(b) in imap]
    te = np.empty(len(keep), M.RATING)
    te["u"], te["i"], te["r"] = [k[0] for k in keep], [k[1] for k in keep], [k[2] for k in keep]
    M.write_binary_ratings(f"{d}/test.bin", te, 600, 300)
    common = ["-k", "64", "-l", "8", "-a", "0.02", "-b", "0.05", "-v", "5", "-seed", "5"]
    out_txt = run([qmf, "-i", f"{d}/train.tsv", "-y", f"{d}/test.tsv", "-o", f"{d}/mt", "-det", "1"] + common)
    out_bin = run([qmf, "-i", f"{d}/train.bin", "-y", f"{d}/test.bin", "-o", f"{d}/mb", "-ob", "1", "-det", "1"] + common)
    rm_txt = [float(e[2]) for e in EPOCH_LINE.findall(out_txt)]
    rm_bin = [float(e[2]) for e in EPOCH_LINE.findall(out_bin)]
    assert len(rm_bin) == 8 and rm_bin == rm_txt, "the same ratings in the same order train to the same RMSE (sequential mode)"
    assert "Num of workers              : 1" in out_bin
    for label in ("Rating histogram", "Grouping", "Matrix reconstruction", "Copy to grouped params", "Additional info init",
                  "Total preprocessing time", "Precision switching", "Total precision switching time", "Error computation time",
                  "Total error computation time", "Parameters update per epoch", "Total parameters update", "Total MF time(ms)"):
        assert re.search(rf"^{re.escape(label)}\s*: [0-9.e+-]+$", out_bin, re.M), label
    ev = run([tmf, "-i", f"{d}/mb.bin", "-y", f"{d}/test.bin", "-v", "5"])
    got = float(re.search(r"RMSE : ([0-9.eE+-]+)", ev).group(1))
    assert abs(got - rm_bin[-1]) <= 1e-6 * rm_bin[-1], "the binary model holds the factors exactly"
    # automatic worker count is printed as a number; no test file: epochs run, the RMSE column is nan
    out = run([qmf, "-i", f"{d}/train.bin"] + common)
    assert re.search(r"^Num of workers              : \d+$", out, re.M) and "Test file                   : None" in out
    assert "The number of test nonzeros : 0" in out
    assert len(re.findall(r"^\d+ [0-9.e-]+ -?nan$", out, re.M)) == 8


def test_two_gpu_run_from_the_command_line(synth, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    d = str(tmp_path)
    write_dataset(synth, d, "train.tsv", "test.tsv")
    for bpg in ("1", "2"):
        out = run([os.path.join(BIN, "quantized_mf"), "-i", f"{d}/train.tsv", "-y", f"{d}/test.tsv", "-o", f"{d}/m{bpg}", "-k", "128", "-l", "10",
                   "-a", "0.02", "-b", "0.015", "-v", "1", "-ug", "8", "-ig", "6", "-s", "0.1", "-it", "2", "-e", "0.5", "-g", "2", "-bpg", bpg])
        rm = [float(e[2]) for e in EPOCH_LINE.findall(out)]
        assert len(rm) == 10 and rm[-1] < rm[0] and np.isfinite(rm).all()
        assert open(f"{d}/m{bpg}_reconst.txt").readline().split() == ["600", "300", "128"]


def test_unimplemented_variants_say_so(synth, tmp_path):
    d = str(tmp_path)
    write_dataset(synth, d, "train.tsv", "test.tsv")
    out = subprocess.run([os.path.join(BIN, "quantized_mf"), "-i", f"{d}/train.tsv", "-y", f"{d}/test.tsv", "-v", "9"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 1 and "unknown training variant" in out.stderr
