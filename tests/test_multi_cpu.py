"""CPU tests (gloo, world_size 2 and 3) of the sharded-training host logic: the partition plan, the
block rotation and the statistics exchange, with a CPU stand-in for the engine that applies the
oracle's update rule.  Nothing here needs a GPU."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def load_multi():
    import importlib.util
    spec = importlib.util.spec_from_file_location("mascot_multi", os.path.join(ROOT, "icdm-2021_mascot_b200", "multi.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


RATING = np.dtype([("r", np.float32), ("u", np.uint32), ("i", np.uint32)])
HYPER = dict(k=64, lr=0.02, decay=0.1, lam=0.015, ug=6, ig=5, sample_ratio=0.3, threshold=0.9, epochs=50, interval=1)


def dataset(seed=5, n_users=150, n_items=90, n=6000):
    rng = np.random.default_rng(seed)
    wu = np.arange(1, n_users + 1) ** -0.8; wi = np.arange(1, n_items + 1) ** -1.0
    R = np.empty(n, RATING)
    R["u"] = rng.choice(n_users, n, p=wu / wu.sum()); R["i"] = rng.choice(n_items, n, p=wi / wi.sum())
    R["u"][:n_users] = np.arange(n_users); R["i"][:n_items] = np.arange(n_items)
    R["r"] = rng.choice(np.arange(0.5, 5.01, 0.5), n)
    R = R[rng.permutation(n)]
    P = (rng.standard_normal((n_users, HYPER["k"])) * 0.2).astype(np.float32)
    Q = (rng.standard_normal((n_items, HYPER["k"])) * 0.2).astype(np.float32)
    test = R[rng.permutation(n)[:800]].copy()
    return R, test, P, Q, n_users, n_items


class OracleShard:
    """CPU stand-in for an engine shard: same interface as multi.EngineShard, oracle arithmetic."""

    def __init__(self, O, multi, plan, rank, train, test, P, Q, n_users, n_items):
        self.O, self.plan, self.rank = O, plan, rank
        k = HYPER["k"]
        mine, seg, my_test = multi.shard_ratings(plan, rank, train, test)
        us = np.argsort(plan.user_degree, kind="stable"); its = np.argsort(plan.item_degree, kind="stable")
        self.u2s = np.empty(n_users, np.uint32); self.u2s[us] = np.arange(n_users, dtype=np.uint32)
        self.i2s = np.empty(n_items, np.uint32); self.i2s[its] = np.arange(n_items, dtype=np.uint32)
        uend, ugof = O.grouping(plan.user_degree[us], HYPER["ug"]); iend, igof = O.grouping(plan.item_degree[its], HYPER["ig"])
        Ps = np.empty_like(P); Ps[self.u2s] = P
        Qs = np.empty_like(Q); Qs[self.i2s] = Q
        self.model = O.MascotModel(k, Ps, Qs, ugof, igof, np.zeros(len(uend), np.uint8), np.zeros(len(iend), np.uint8))
        self.R = mine.copy(); self.R["u"] = self.u2s[mine["u"]]; self.R["i"] = self.i2s[mine["i"]]
        self.seg = seg.astype(np.int64)
        t = my_test[np.lexsort((my_test["i"], my_test["u"]))]
        self.T = t.copy(); self.T["u"] = self.u2s[t["u"]]; self.T["i"] = self.i2s[t["i"]]
        self.lrs = O.lr_schedule(HYPER["lr"], HYPER["decay"], HYPER["epochs"])
        self.rules = O.rules_reference()
        self.init_u = np.ones(len(uend), np.float32); self.init_i = np.ones(len(iend), np.float32)
        self.stats = None
        self.processed = 0

    def block_tensors(self, b):
        # strided views of raw bytes [rows of the block, bytes per row], like the device views of the real
        # engine; as there, an arena travels only while it holds live rows (a row lives in exactly one)
        n, w = self.model.Q16.shape[0], self.plan.blocks
        views = []
        if (self.model.iprec == 0).any():
            views.append(torch.from_numpy(self.model.Q16.view(np.uint8).reshape(n, -1))[b::w])
        if (self.model.iprec != 0).any():
            views.append(torch.from_numpy(self.model.Q32.view(np.uint8).reshape(n, -1))[b::w])
        return views

    def is_check_epoch(self, epoch):
        return self.O.is_check_epoch(epoch, HYPER["epochs"], HYPER["interval"])

    def stats_begin(self):
        k, ug, ig = HYPER["k"], len(self.model.uprec), len(self.model.iprec)
        self.stats = [np.zeros(ug * k, np.float32), np.zeros(ig * k, np.float32), np.zeros(ug, np.float32), np.zeros(ig, np.float32)]

    def train_segment(self, epoch, b, collect_stats=False):
        lo, hi = int(self.seg[b]), int(self.seg[b + 1])
        if hi <= lo:
            return
        n = hi - lo
        fsp = n - min(int(np.float32(n) * np.float32(HYPER["sample_ratio"])), n) if collect_stats else None
        self.model.run(self.R[lo:hi], None, float(self.lrs[epoch]), HYPER["lam"], self.rules, first_sample_pos=fsp,
                       stats=collect_stats, item_stats_by_run=True, into=self.stats if collect_stats else None)
        self.processed += n

    def sync(self):
        pass

    def device_order(self):
        import contextlib
        return contextlib.nullcontext()

    def stats_fetch(self):
        return [a.copy() for a in self.stats]

    def stats_apply(self, epoch, gp, gq, np_, nq):
        O, k = self.O, HYPER["k"]
        eu = O.group_errors(gp, np_, k, self.model.uprec, self.init_u)
        ei = O.group_errors(gq, nq, k, self.model.iprec, self.init_i)
        pu = pi = 0
        if epoch == 5:
            self.init_u, self.init_i = eu.copy(), ei.copy()
        elif epoch > 5:
            for g in range(len(eu)):
                if eu[g] > HYPER["threshold"] and not self.model.uprec[g]:
                    self.model.promote("u", g); pu += 1
            for g in range(len(ei)):
                if ei[g] > HYPER["threshold"] and not self.model.iprec[g]:
                    self.model.promote("i", g); pi += 1
        return pu, pi

    def eval_sq_error(self):
        P, Q = self.model.factors()
        pred = np.einsum("nk,nk->n", P[self.T["u"]].astype(np.float64), Q[self.T["i"]].astype(np.float64))
        return float(((self.T["r"] - pred) ** 2).sum()), int(self.T.size)


def load_binding():
    """ctypes binding of libmascot (used here only for the device-free schedule function)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("mascot_binding", os.path.join(ROOT, "icdm-2021_mascot_b200", "mascot.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def library_schedule(world, per_gpu):
    """The library's own block schedule (mascot_shard_schedule), as the callable multi.train_epoch takes."""
    M = load_binding()
    return lambda rank, step: M.shard_schedule(world, per_gpu, rank, step)


def _worker(rank, world, port, out_dir, per_gpu=1):
    import oracle as O
    multi = load_multi()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        R, test, P, Q, n_users, n_items = dataset()
        plan = multi.make_plan(R["u"], R["i"], n_users, n_items, world, world * per_gpu)
        shard = OracleShard(O, multi, plan, rank, R, test, P, Q, n_users, n_items)
        rm, promoted = [], []
        for e in range(8):
            _, pr = multi.train_epoch(dist, shard, rank, world, e, schedule=library_schedule(world, per_gpu))
            multi.gather_item_factors(dist, shard, world)
            rm.append(multi.global_rmse(dist, shard, world))
            promoted.append(pr)
        Pm, Qm = shard.model.factors()
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), P=Pm, Q=Qm, rmse=np.array(rm), promoted=np.array(promoted),
                 processed=shard.processed, uprec=shard.model.uprec, iprec=shard.model.iprec,
                 mine=(plan.user_rank == rank))
    finally:
        dist.destroy_process_group()


def _toy_worker(rank, world, port, out_dir):
    """Rotation only: every rank adds rank+1 to whatever block it holds in each sub-epoch."""
    multi = load_multi()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        rows = [(0, 3), (3, 4), (4, 9), (9, 9), (9, 12)][:world] if world <= 5 else None
        data = torch.zeros(12, 4)
        visits = torch.zeros(12, 4)

        class Toy:
            def block_tensors(self, b):
                lo, hi = rows[b]
                return [data[lo:hi], visits[lo:hi]]
        toy = Toy()
        for s in range(world):
            b = (rank + s) % world
            lo, hi = rows[b]
            data[lo:hi] += rank + 1
            visits[lo:hi] += 1
            multi.exchange_block(dist, toy, b, (rank + s + 1) % world, (rank - 1) % world, (rank + 1) % world)
        lo, hi = rows[rank]
        torch.save({"data": data[lo:hi].clone(), "visits": visits[lo:hi].clone()}, os.path.join(out_dir, f"toy{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_blocks_visit_every_rank_once_and_return_home(tmp_path, world):
    mp.spawn(_toy_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        got = torch.load(os.path.join(tmp_path, f"toy{rank}.pt"))
        assert (got["visits"] == world).all(), "home block was held by every rank exactly once"
        assert (got["data"] == world * (world + 1) / 2).all()


def test_plan_is_a_partition_with_balanced_users():
    multi = load_multi()
    R, test, P, Q, n_users, n_items = dataset()
    for world in (1, 2, 4, 8):
        plan = multi.make_plan(R["u"], R["i"], n_users, n_items, world)
        assert plan.item_block.min() == 0 and plan.item_block.max() == world - 1
        total = 0
        for rank in range(world):
            mine, seg, my_test = multi.shard_ratings(plan, rank, R, test)
            total += mine.size
            assert seg[0] == 0 and seg[-1] == mine.size and (np.diff(seg.astype(np.int64)) >= 0).all()
            for b in range(world):
                rows = plan.item_sorted_index[mine["i"][int(seg[b]):int(seg[b + 1])]]
                assert (rows % world == b).all()
        # every block gets about the same number of ratings (same mix of popular and rare items)
        per_block = np.bincount(plan.item_block[R["i"]], minlength=world)
        assert per_block.max() <= 1.25 * per_block.mean() + plan.item_degree.max()
        assert total == R.size
        per_rank = np.bincount(plan.user_rank[R["u"]], minlength=world)
        assert per_rank.max() <= 1.25 * per_rank.mean() + plan.user_degree.max()


def sequential_replay(O, multi, world, per_gpu, epochs=8):
    """The sharded run in ONE process: `world` stand-in shards, the library's block order, the hand-overs
    emulated by copying blocks between the shards.  Returns (shards, plan, rmse per epoch)."""
    R, test, P, Q, n_users, n_items = dataset()
    blocks = world * per_gpu
    plan = multi.make_plan(R["u"], R["i"], n_users, n_items, world, blocks)
    shards = [OracleShard(O, multi, plan, r, R, test, P, Q, n_users, n_items) for r in range(world)]

    def copy_block(src, dst, b):
        for a, c in zip(src.block_tensors(b), dst.block_tensors(b)):
            c.copy_(a)
    rm = []
    for e in range(epochs):
        check = shards[0].is_check_epoch(e)
        if check:
            for sh in shards:
                sh.stats_begin()
        for s in range(blocks):
            for r in range(world):
                shards[r].train_segment(e, (per_gpu * r + s) % blocks, collect_stats=check)
            for r in range(world):
                if world > 1:
                    copy_block(shards[r], shards[(r - 1) % world], (per_gpu * r + s) % blocks)
        if check:
            sums = [sum(sh.stats_fetch()[j] for sh in shards) for j in range(4)]
            for sh in shards:
                sh.stats_apply(e, *sums)
        for b in range(blocks):
            for r in range(world):
                if r != b // per_gpu:
                    copy_block(shards[b // per_gpu], shards[r], b)
        parts = [sh.eval_sq_error() for sh in shards]
        rm.append(np.sqrt(sum(p[0] for p in parts) / sum(p[1] for p in parts)))
    return shards, plan, rm


@pytest.mark.parametrize("per_gpu", [1, 2])
def test_two_ranks_equal_the_sequential_replay_bit_for_bit(tmp_path, per_gpu):
    import oracle as O
    multi = load_multi()
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), per_gpu), nprocs=world, join=True)
    got = [np.load(os.path.join(tmp_path, f"rank{r}.npz")) for r in range(world)]
    R, test, P, Q, n_users, n_items = dataset()
    assert sum(int(g["processed"]) for g in got) == 8 * R.size, "every rating exactly once per epoch"
    # sequential replay of the same block order in ONE process
    shards, plan, rm = sequential_replay(O, multi, world, per_gpu)
    for r in range(world):
        Pm, Qm = shards[r].model.factors()
        mine_rows = shards[r].u2s[np.flatnonzero(plan.user_rank == r)]
        assert (got[r]["P"][mine_rows].view(np.uint32) == Pm[mine_rows].view(np.uint32)).all()
        assert (got[r]["Q"].view(np.uint32) == Qm.view(np.uint32)).all()
        assert (got[r]["uprec"] == shards[r].model.uprec).all() and (got[r]["iprec"] == shards[r].model.iprec).all()
        assert np.allclose(got[r]["rmse"], rm, rtol=1e-12)
    assert (got[0]["Q"].view(np.uint32) == got[1]["Q"].view(np.uint32)).all(), "Q is identical on both ranks after the gather"
    assert got[0]["promoted"].sum() > 0, "the case is meant to exercise switching across ranks"
    assert got[0]["rmse"][-1] < got[0]["rmse"][0]


@pytest.mark.parametrize("world,per_gpu", [(1, 1), (1, 2), (2, 1), (2, 2), (3, 1), (4, 2), (8, 1), (8, 2)])
def test_library_schedule_is_conflict_free_and_complete(world, per_gpu):
    """mascot_shard_schedule (pure host function of libmascot): in every step the ranks train distinct
    blocks; over an epoch every rank trains every block exactly once; a block is sent to rank-1 and the
    block that arrives is the one rank+1 trained in the same step and is trained here `per_gpu` steps
    later, so with two blocks per GPU a block in flight is never the one being trained."""
    M = load_binding()
    blocks = world * per_gpu
    seen = {r: [] for r in range(world)}
    for step in range(blocks):
        row = [M.shard_schedule(world, per_gpu, r, step) for r in range(world)]
        trained = [x[0] for x in row]
        assert len(set(trained)) == world, "no two ranks hold the same block"
        for r, (b, dst, incoming, src) in enumerate(row):
            assert dst == (r - 1) % world and src == (r + 1) % world
            assert incoming == row[src][0], "what arrives is what the neighbour has just trained"
            later = M.shard_schedule(world, per_gpu, r, (step + per_gpu) % blocks)[0]
            assert later == incoming
            if per_gpu == 2 and world > 1:
                assert M.shard_schedule(world, per_gpu, r, (step + 1) % blocks)[0] not in (incoming, b)
            seen[r].append(b)
    for r in range(world):
        assert sorted(seen[r]) == list(range(blocks))
    with pytest.raises(M.MascotError):
        M.shard_schedule(world, per_gpu, world, 0)


def _timeout_worker(rank, world, port, out_dir):
    """Rank 1 leaves before the hand-over of the first step; rank 0's bounded wait must end with the
    timeout status instead of blocking."""
    import datetime
    multi = load_multi()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=3))
    status = 0
    try:
        data = torch.zeros(8, 4)

        class Toy:
            def block_tensors(self, b):
                return [data[4 * b:4 * b + 4]]
        if rank == 0:
            try:
                multi.exchange_block(dist, Toy(), 0, 1, 1, 1)          # its partner never sends
            except Exception:
                status = -6                                            # MASCOT_ERR_TIMEOUT
        with open(os.path.join(out_dir, f"status{rank}.txt"), "w") as f:
            f.write(str(status))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_ends_in_the_timeout_status(tmp_path):
    """Host-made failure: a rank that skips its send.  The waiting rank gives up after the group's limit
    and reports MASCOT_ERR_TIMEOUT (-6); nothing hangs."""
    mp.spawn(_timeout_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(os.path.join(tmp_path, "status0.txt")).read() == "-6"
    assert open(os.path.join(tmp_path, "status1.txt")).read() == "0"
