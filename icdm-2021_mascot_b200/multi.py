"""Sharded (multi-GPU) training on top of the libmascot building blocks: one process per GPU.

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

The schedule and the exchange are written against a tiny shard interface, so the same code drives
libmascot engines on GPUs and a CPU stand-in in the tests.
"""
import numpy as np


class Plan:
    """Who owns which user and which item block an item belongs to."""

    def __init__(self, world, user_rank, item_block, user_degree, item_degree, item_sorted_index):
        self.world = world
        self.user_rank = user_rank                # [n_users] compact id -> rank
        self.item_block = item_block              # [n_items] compact id -> block (= sorted index mod world)
        self.user_degree = user_degree
        self.item_degree = item_degree
        self.item_sorted_index = item_sorted_index


def make_plan(train_u, train_i, n_users, n_items, world):
    """Degree tables of the whole training set, user dealing and item blocks."""
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
    item_block = (item_sorted_index % np.uint32(world)).astype(np.int32)
    return Plan(world, user_rank, item_block, user_degree, item_degree, item_sorted_index)


def shard_ratings(plan, rank, train, test):
    """The ratings of this rank's users, ordered into one segment per item block."""
    mine = train[plan.user_rank[train["u"]] == rank]
    blk = plan.item_block[mine["i"]]
    order = np.argsort(blk, kind="stable")
    mine = np.ascontiguousarray(mine[order])
    counts = np.bincount(blk, minlength=plan.world)
    seg = np.zeros(plan.world + 1, np.uint64)
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


def train_epoch(dist, shard, rank, world, epoch, comm_device="cpu"):
    """One epoch = `world` sub-epochs with a block rotation after each.  Returns bytes sent."""
    import torch
    check = shard.is_check_epoch(epoch)
    sent = 0
    with shard.device_order():
        if check:
            shard.stats_begin()
        for s in range(world):
            b = (rank + s) % world
            shard.train_segment(epoch, b, collect_stats=check)
            if world > 1:
                sent += exchange_block(dist, shard, b, (rank + s + 1) % world, (rank - 1) % world, (rank + 1) % world)
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
    with shard.device_order():
        for b in range(world):
            for t in shard.block_tensors(b):
                buf = t.contiguous()
                dist.broadcast(buf, src=b)
                t.copy_(buf)
    shard.sync()


def global_rmse(dist, shard, world, comm_device="cpu"):
    import torch
    s, n = shard.eval_sq_error()
    t = torch.tensor([s, float(n)], dtype=torch.float64, device=comm_device)
    if world > 1:
        dist.all_reduce(t)
    return float(torch.sqrt(t[0] / t[1]).item()) if t[1] > 0 else float("nan")


class _DeviceBytes:
    """Raw device memory exposed through the CUDA array interface, so torch can wrap it without a copy."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


class EngineShard:
    """A libmascot engine holding one rank's shard."""

    def __init__(self, M, cfg, plan, rank, train, test, n_users, n_items):
        import torch
        self.M, self.plan, self.rank = M, plan, rank
        mine, seg, my_test = shard_ratings(plan, rank, train, test)
        self.n_local = int(mine.size)
        self.local_ratings = mine                   # host copy of this rank's ratings, in segment order
        self.n_items = int(n_items)
        self.engine = M.Engine(cfg)
        self.engine.set_ratings_sharded(mine, seg, my_test, n_users, n_items, plan.user_degree, plan.item_degree)
        self.device = torch.device("cuda", int(cfg.device))
        self.stream = torch.cuda.ExternalStream(self.engine.stream_handle(), device=self.device)
        self._views = {}
        self._live = None

    def device_order(self):
        """Context in which torch's current stream is the engine's stream."""
        import torch
        return torch.cuda.stream(self.stream)

    def _live_arenas(self):
        """(binary16 arena holds live item rows, fp32 arena holds live item rows): an item row lives in
        exactly one of them, by its group's precision, so an arena without live rows need not travel.
        Every rank reaches the same answer, because all take the same switching decisions."""
        if self._live is None:
            prec = self.engine.group_info(1)[1]
            self._live = (bool((prec == 0).any()), bool((prec != 0).any()))
        return self._live

    def block_tensors(self, b):
        """Strided byte views [rows of block b, bytes per row] of the item arenas that hold live rows."""
        import torch
        if b not in self._views:
            views = []
            for live, (ptr, nbytes) in zip(self._live_arenas(), self.engine.item_rows(0, self.n_items)):
                if live and ptr and nbytes:
                    whole = torch.as_tensor(_DeviceBytes(ptr, nbytes), device=self.device).view(self.n_items, nbytes // self.n_items)
                    views.append(whole[b::self.plan.world])
            self._views[b] = views
        return self._views[b]

    def is_check_epoch(self, epoch):
        return self.engine.is_check_epoch(epoch)

    def stats_begin(self):
        self.engine.stats_begin()

    def train_segment(self, epoch, b, collect_stats=False):
        self.engine.train_segment(epoch, b, collect_stats, wait=False)

    def sync(self):
        self.engine.sync()

    def stats_fetch(self):
        return self.engine.stats_fetch()

    def stats_apply(self, epoch, *sums):
        promoted = self.engine.stats_apply(epoch, *sums)
        if promoted[1]:
            self._live = None                     # item groups changed precision: re-derive which arenas travel
            self._views.clear()
        return promoted

    def eval_sq_error(self):
        return self.engine.eval_sq_error()

    def close(self):
        self._views.clear()
        self.engine.close()
