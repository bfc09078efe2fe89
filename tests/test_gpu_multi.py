"""GPU test of the sharded path on 2 GPUs (skipped on a single-GPU box): two libmascot engines in
deterministic mode, item blocks exchanged with NCCL send/recv, must equal the sequential CPU replay
of the same block order bit for bit."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_gpus_equal_the_sequential_replay(tmp_path, oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_multi_cpu import OracleShard, dataset, load_multi
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", os.path.join(ROOT, "tests", "multi_gpu_worker.py"), str(tmp_path)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    got = [np.load(os.path.join(tmp_path, f"gpu_rank{r}.npz")) for r in range(2)]
    multi = load_multi()
    world = 2
    R, test, P, Q, n_users, n_items = dataset()
    plan = multi.make_plan(R["u"], R["i"], n_users, n_items, world)
    shards = [OracleShard(oracle, multi, plan, r, R, test, P, Q, n_users, n_items) for r in range(world)]

    def copy_block(src, dst, b):
        for a, c in zip(src.block_tensors(b), dst.block_tensors(b)):
            c.copy_(a)
    for e in range(8):
        check = shards[0].is_check_epoch(e)
        if check:
            for sh in shards:
                sh.stats_begin()
        for s in range(world):
            for r in range(world):
                shards[r].train_segment(e, (r + s) % world, collect_stats=check)
            for r in range(world):
                copy_block(shards[r], shards[(r - 1) % world], (r + s) % world)
        if check:
            sums = [sum(sh.stats_fetch()[j] for sh in shards) for j in range(4)]
            for sh in shards:
                sh.stats_apply(e, *sums)
        for b in range(world):
            for r in range(world):
                if r != b:
                    copy_block(shards[b], shards[r], b)
    for r in range(world):
        Pm, Qm = shards[r].model.factors()
        rows = shards[r].u2s[np.flatnonzero(plan.user_rank == r)]
        assert (got[r]["P"][rows].view(np.uint32) == Pm[rows].view(np.uint32)).all(), f"rank {r} user factors"
        assert (got[r]["Q"].view(np.uint32) == Qm.view(np.uint32)).all(), f"rank {r} item factors"
        assert (got[r]["uprec"] == shards[r].model.uprec).all() and (got[r]["iprec"] == shards[r].model.iprec).all()
    assert got[0]["promoted"].sum() > 0
