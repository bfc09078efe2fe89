"""GPU tests of the library's sharded path (mascot_shard_*, csrc/shard.cu): engines in deterministic
mode, item blocks handed over by the C++ schedule with NCCL, must equal the sequential CPU replay of the
same block order bit for bit.  The one-GPU case runs everywhere; the two-GPU cases are skipped on a
single-GPU box."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_ranks(tmp_path, world, per_gpu):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "multi_gpu_worker.py"), str(tmp_path), str(r), str(world), str(per_gpu)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r}:\n" + outs[r][-3000:]
    return [np.load(os.path.join(tmp_path, f"gpu_rank{r}.npz")) for r in range(world)]


def check_against_replay(oracle, got, world, per_gpu):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_multi_cpu import dataset, load_multi, sequential_replay
    multi = load_multi()
    shards, plan, rm = sequential_replay(oracle, multi, world, per_gpu)
    R, test, P, Q, n_users, n_items = dataset()
    assert sum(int(g["local"]) for g in got) == R.size, "every rating belongs to exactly one rank"
    for r in range(world):
        assert np.array_equal(got[r]["u2s"], shards[r].u2s) and np.array_equal(got[r]["i2s"], shards[r].i2s)
        assert int(got[r]["local"]) == int((plan.user_rank[R["u"]] == r).sum()), "the library deals the users like the plan"
        Pm, Qm = shards[r].model.factors()
        # after the gather every rank holds the whole model: each user's rows from the rank that owns it
        for owner in range(world):
            rows = shards[owner].u2s[np.flatnonzero(plan.user_rank == owner)]
            Po, _ = shards[owner].model.factors()
            assert (got[r]["P"][rows].view(np.uint32) == Po[rows].view(np.uint32)).all(), f"rank {r}: user rows of rank {owner}"
        assert (got[r]["Q"].view(np.uint32) == Qm.view(np.uint32)).all(), f"rank {r} item factors"
        assert (got[r]["uprec"] == shards[r].model.uprec).all() and (got[r]["iprec"] == shards[r].model.iprec).all()
        # the engine sums float32 block partials, the replay float64 squared errors: 1e-6 relative
        assert np.allclose(got[r]["rmse"], rm, rtol=1e-6), (got[r]["rmse"], rm)
        want_t = shards[r].T
        key = lambda a: np.lexsort((a["r"].view(np.uint32), a["i"], a["u"]))
        assert np.array_equal(got[r]["test_ratings"][key(got[r]["test_ratings"])], want_t[key(want_t)])
    assert got[0]["promoted"].sum() > 0, "the case is meant to exercise switching"
    assert got[0]["rmse"][-1] < got[0]["rmse"][0]
    if world > 1:
        assert all(int(g["sent"]) > 0 for g in got)


@pytest.mark.parametrize("per_gpu", [1, 2])
def test_group_of_one_equals_the_sequential_replay(tmp_path, oracle, per_gpu):
    """world = 1: the set-up selection, the block-contiguous item layout (two blocks when per_gpu = 2), the
    step loop and the statistics path of the sharded code, without a second GPU."""
    got = run_ranks(tmp_path, 1, per_gpu)
    check_against_replay(oracle, got, 1, per_gpu)


@pytest.mark.parametrize("per_gpu", [1, 2])
def test_two_gpus_equal_the_sequential_replay(tmp_path, oracle, per_gpu):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    got = run_ranks(tmp_path, 2, per_gpu)
    check_against_replay(oracle, got, 2, per_gpu)
    assert (got[0]["Q"].view(np.uint32) == got[1]["Q"].view(np.uint32)).all()
    assert (got[0]["P"].view(np.uint32) == got[1]["P"].view(np.uint32)).all()
