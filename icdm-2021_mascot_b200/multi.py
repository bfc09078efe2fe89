"""Host-side model of sharded (multi-GPU) training, kept as a TEST DRIVER: the product path is the C++
implementation inside libmascot (csrc/shard.cu, mascot_shard_* in include/mascot.h).  This module
restates its partition plan and its block rotation in Python, so that CPU tests can run the schedule
with gloo ranks and a CPU stand-in for the engine, and so that GPU tests have an independent replay to
compare the library against.

Scheme (the reference is single-GPU; this has no counterpart there): the users are dealt to the
ranks so that every rank gets the same mix of degrees, and with them their ratings and their rows of
P; the items - in the engine's degree-sorted index space - are dealt round-robin into `world` blocks
(row r belongs to block r mod world), so that every block holds the same mix of popular and rare
items: the ranks then take the same time for a sub-epoch whichever block they hold, and no rank
ever has all its workers on a handful of very popular rows.  Sub-epoch s: rank g trains its ratings that fall into item block
(g + s) mod world, then hands that block of Q to rank g-1 and receives block (g + s + 1) mod world
from rank g+1.  At any time the ranks work on disjoint users AND disjoint items, so there are no
races between GPUs, and after `world` sub-epochs every block is back home.  The only data-path
communication is that block hand-over (point-to-point, NCCL send/recv through torch.distributed on
GPUs); the small g-switching statistics and the RMSE partial sums are all-reduced.

With `blocks` = 2 x world the library's overlapped variant is modelled: rank g trains block
(2 g + t) mod blocks in step t and a block is trained by its receiver two steps after it was sent.

The schedule and the exchange are written against a tiny shard interface (see tests/test_multi_cpu.py).
"""
import numpy as np


class Plan:
    """Who owns which user and which item block an item belongs to."""

    def __init__(self, world, user_rank, item_block, user_degree, item_degree, item_sorted_index, blocks=None):
        self.world = world
        self.blocks = blocks or world             # item blocks in all (world x blocks per GPU)
        self.user_rank = user_rank                # [n_users] compact id -> rank
        self.item_block = item_block              # [n_items] compact id -> block (= sorted index mod world)
        self.user_degree = user_degree
        self.item_degree = item_degree
        self.item_sorted_index = item_sorted_index


def make_plan(train_u, train_i, n_users, n_items, world, blocks=None):
    """Degree tables of the whole training set, user dealing and item blocks."""
    blocks = blocks or world
    user_degree = np.bincount(train_u, minlength=n_users).astype(np.uint32)
    item_degree = np.bincount(train_i, minlength=n_items).astype(np.uint32)
    # same order as the engine's set-up: ascending degree, ties by ascending id
    user_sorted = np.argsort(user_degree, kind="stable")
    item_sorted = np.argsort(item_degree, kind="stable")
    # deal the users out from the heaviest down, reversing direction every round (snake order), so
    # that the rating counts of the ranks stay close even for heavy-tailed degrees
    pos = np.arange(n_users)
    rnd, idx = pos // world, pos % world
    user_rank = np.empty(n_users, np.int32)
    user_rank[user_sorted[::-1]] = np.where(rnd % 2 == 0, idx, world - 1 - idx)
    item_sorted_index = np.empty(n_items, np.uint32)
    item_sorted_index[item_sorted] = np.arange(n_items, dtype=np.uint32)
    item_block = (item_sorted_index % np.uint32(blocks)).astype(np.int32)
    return Plan(world, user_rank, item_block, user_degree, item_degree, item_sorted_index, blocks)


def shard_ratings(plan, rank, train, test):
    """The ratings of this rank's users, ordered into one segment per item block."""
    mine = train[plan.user_rank[train["u"]] == rank]
    blk = plan.item_block[mine["i"]]
    order = np.argsort(blk, kind="stable")
    mine = np.ascontiguousarray(mine[order])
    counts = np.bincount(blk, minlength=plan.blocks)
    seg = np.zeros(plan.blocks + 1, np.uint64)
    seg[1:] = np.cumsum(counts)
    my_test = np.ascontiguousarray(test[plan.user_rank[test["u"]] == rank])
    return mine, seg, my_test


def workers_per_rank(n_train_global, world):
    """Concurrent sequential workers per GPU (`mascot_config.num_workers`) for a sharded run.

    What decides the convergence per epoch of these racy updates is how many workers touch one row at
    the same time.  A rank puts all its workers on 1/world of the items (and of the users), so a row
    sees `world` times the per-rank count: the total over all ranks is what has to stay bounded, not
    the count per GPU.  Measured on the 100M-rating configuration, a total of about twice the
    single-GPU automatic choice (n/8192) still ends within the tolerance of the reference's final
    RMSE and four times does not; 1.5 times is used."""
    total = max(3 * int(n_train_global) // 16384, 512)
    return max(total // world, 64)


def exchange_block(dist, shard, send_block, recv_block, dst, src):
    """Hand `send_block` to rank dst and take `recv_block` from rank src (in place, both arenas).

    A block is a strided set of rows, so it is packed into a contiguous buffer for the transfer and
    unpacked on arrival.  On GPUs the caller has made the engine's stream the current one
    (shard.device_order()), so packing and transfer start when the kernel queued before them has
    finished and the next kernel waits for the unpacking: the ordering is done by the device, the
    host never waits."""
    import torch
    if send_block == recv_block and dst == src:
        return 0
    ops, nbytes = [], 0
    for t in shard.block_tensors(send_block):
        packed = t.contiguous()
        ops.append(dist.P2POp(dist.isend, packed, dst))
        nbytes += packed.numel() * packed.element_size()
    arriving = []
    for t in shard.block_tensors(recv_block):
        buf = torch.empty(t.shape, dtype=t.dtype, device=t.device)
        ops.append(dist.P2POp(dist.irecv, buf, src))
        arriving.append((t, buf))
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    for t, buf in arriving:
        t.copy_(buf)
    return nbytes


def train_epoch(dist, shard, rank, world, epoch, comm_device="cpu", schedule=None):
    """One epoch = `blocks` steps with a block hand-over after each.  `schedule(rank, step)` returns
    (block trained, rank it goes to, block that arrives, rank it comes from); default: one block per
    rank.  Returns bytes sent."""
    import torch
    check = shard.is_check_epoch(epoch)
    sent = 0
    steps = getattr(getattr(shard, "plan", None), "blocks", world) if schedule else world
    if schedule is None:
        schedule = lambda r, s: ((r + s) % world, (r - 1) % world, (r + s + 1) % world, (r + 1) % world)
    with shard.device_order():
        if check:
            shard.stats_begin()
        for s in range(steps):
            b, dst, incoming, src = schedule(rank, s)
            shard.train_segment(epoch, b, collect_stats=check)
            if world > 1:
                sent += exchange_block(dist, shard, b, incoming, dst, src)
        promoted = (0, 0)
        if check:
            parts = shard.stats_fetch()
            if world > 1:
                # one message for the four arrays
                flat = torch.from_numpy(np.concatenate([np.asarray(a, np.float32).reshape(-1) for a in parts])).to(comm_device)
                dist.all_reduce(flat)
                flat = flat.cpu().numpy()
                cuts = np.cumsum([0] + [a.size for a in parts])
                parts = [flat[cuts[j]:cuts[j + 1]] for j in range(len(parts))]
            promoted = shard.stats_apply(epoch, *parts)
    return sent, promoted


def gather_item_factors(dist, shard, world):
    """After an epoch every rank holds only its home block fresh; make all of Q fresh everywhere."""
    if world == 1:
        return
    blocks = getattr(getattr(shard, "plan", None), "blocks", world)
    per_rank = blocks // world
    with shard.device_order():
        for b in range(blocks):
            for t in shard.block_tensors(b):
                buf = t.contiguous()
                dist.broadcast(buf, src=b // per_rank)     # the home of block b
                t.copy_(buf)
    shard.sync()


def global_rmse(dist, shard, world, comm_device="cpu"):
    import torch
    s, n = shard.eval_sq_error()
    t = torch.tensor([s, float(n)], dtype=torch.float64, device=comm_device)
    if world > 1:
        dist.all_reduce(t)
    return float(torch.sqrt(t[0] / t[1]).item()) if t[1] > 0 else float("nan")
