"""ctypes binding of libmascot.so - the thin Python face of the C ABI in include/mascot.h.

Used by the tests, the benchmark and the smoke test; the production host code is the C++
command line (cli/quantized_mf.cpp, cli/test_mf.cpp).  There is no fallback: if the shared library
is missing or no CUDA device is usable, calls raise.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MASCOT_LIB_PATH", os.path.join(HERE, "libmascot.so"))

RATING = np.dtype([("r", np.float32), ("u", np.uint32), ("i", np.uint32)])

V_MASCOT, V_AFP, V_MUPPET, V_MPT, V_SGD, V_NAIVE, V_MEMQUANT, V_SWITCH_ONLY = 1, 2, 3, 4, 5, 6, 7, 8

OK, ERR_BAD_ARG, ERR_CUDA, ERR_OOM, ERR_STATE, ERR_NO_DEVICE, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_COMM = \
    0, -1, -2, -3, -4, -5, -6, -7, -8

EXPORTS = [
    "mascot_abi_info", "mascot_config_default", "mascot_create", "mascot_destroy", "mascot_last_error", "mascot_status_string",
    "mascot_set_ratings", "mascot_init_factors", "mascot_set_factors", "mascot_train_epoch", "mascot_eval_rmse",
    "mascot_get_factors", "mascot_get_group_info", "mascot_get_index_maps", "mascot_get_sample_stats",
    "mascot_get_test_ratings", "mascot_promote_group", "mascot_reload_train", "mascot_stream_source_index", "mascot_get_stream_order", "mascot_rmse_host", "mascot_rmse_device", "mascot_rmse_device_noalloc",
    "mascot_set_ratings_sharded", "mascot_is_check_epoch", "mascot_stats_begin", "mascot_train_segment", "mascot_stats_fetch",
    "mascot_stats_apply", "mascot_item_rows", "mascot_sync", "mascot_get_stream", "mascot_eval_sq_error", "mascot_train_epoch_streamed",
    "mascot_release_scratch", "mascot_comm_unique_id", "mascot_shard_init", "mascot_shard_set_ratings", "mascot_shard_train_epoch",
    "mascot_shard_eval_rmse", "mascot_shard_gather_factors", "mascot_shard_info", "mascot_shard_schedule", "mascot_probe_read_bandwidth", "mascot_get_timings", "mascot_get_worker_count",
]

COMM_ID_BYTES = 128


class Config(C.Structure):
    _fields_ = [
        ("lambda_", C.c_float), ("learning_rate", C.c_float), ("decay", C.c_float), ("sample_ratio", C.c_float),
        ("error_threshold", C.c_float), ("interval", C.c_uint32), ("user_group_num", C.c_uint32),
        ("item_group_num", C.c_uint32), ("k", C.c_uint32), ("num_workers", C.c_uint32), ("epoch", C.c_uint32),
        ("thread_block_size", C.c_uint32), ("version", C.c_uint32), ("is_yahoo", C.c_uint32),
        ("deterministic", C.c_uint32), ("shuffle", C.c_uint32), ("seed", C.c_uint64), ("device", C.c_int32),
        ("muppet_width", C.c_uint32), ("plain_user_stores", C.c_uint32), ("l2_item_window", C.c_uint32), ("no_class_partition", C.c_uint32), ("run_window_log2", C.c_uint32), ("reserved", C.c_uint32 * 2),
    ]


class EpochStats(C.Structure):
    _fields_ = [
        ("updates", C.c_uint64), ("lr", C.c_float), ("kernel_ms", C.c_float), ("total_ms", C.c_float),
        ("error_check", C.c_uint32), ("promoted_user_groups", C.c_uint32), ("promoted_item_groups", C.c_uint32),
        ("kernel_launches", C.c_uint32), ("workers", C.c_uint32), ("pass_bits", C.c_uint32),
        ("algorithmic_bytes", C.c_uint64),
    ]


class MascotError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"libmascot status {status}: {message}")
        self.status = status


_lib = None


def load():
    """dlopen libmascot.so (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is missing - run `python icdm-2021_mascot_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        L.mascot_last_error.restype = C.c_char_p
        L.mascot_last_error.argtypes = [C.c_void_p]
        L.mascot_status_string.restype = C.c_char_p
        L.mascot_status_string.argtypes = [C.c_int]
        ver, csz, ssz = C.c_uint32(), C.c_uint32(), C.c_uint32()
        L.mascot_abi_info(C.byref(ver), C.byref(csz), C.byref(ssz))
        if (csz.value, ssz.value) != (C.sizeof(Config), C.sizeof(EpochStats)):
            raise OSError(f"libmascot ABI mismatch: library structs are {csz.value}/{ssz.value} bytes, "
                          f"binding expects {C.sizeof(Config)}/{C.sizeof(EpochStats)}")
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def default_config(**overrides):
    cfg = Config()
    load().mascot_config_default(C.byref(cfg))
    for key, val in overrides.items():
        setattr(cfg, "lambda_" if key in ("lambda", "lam") else key, val)
    return cfg


def as_ratings(a):
    a = np.ascontiguousarray(a)
    if a.dtype != RATING:
        a = a.reshape(-1, 3).astype(np.uint32, copy=False).view(RATING).reshape(-1)
    return a


def make_ratings(u, i, r):
    out = np.empty(len(r), RATING)
    out["u"], out["i"], out["r"] = u, i, r
    return out


class Engine:
    """One libmascot handle."""

    def __init__(self, cfg):
        self._lib = load()
        self.cfg = cfg
        self._h = C.c_void_p()
        rc = self._lib.mascot_create(C.byref(cfg), C.byref(self._h))
        if rc != OK:
            raise MascotError(rc, self._lib.mascot_last_error(None).decode())
        self.k = int(cfg.k)
        self.n_users = self.n_items = 0
        self.n_train = self.n_test = 0

    def _check(self, rc):
        if rc != OK:
            raise MascotError(rc, self._lib.mascot_last_error(self._h).decode())

    def close(self):
        if self._h:
            self._lib.mascot_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_ratings(self, train, test, n_users, n_items):
        train, test = as_ratings(train), as_ratings(test)
        self._check(self._lib.mascot_set_ratings(self._h, _ptr(train), C.c_uint64(train.size), _ptr(test),
                                                 C.c_uint64(test.size), C.c_uint32(n_users), C.c_uint32(n_items)))
        self.n_users, self.n_items, self.n_train, self.n_test = n_users, n_items, train.size, test.size

    def set_ratings_raw(self, train_ptr, n_train, test_ptr, n_test, n_users, n_items):
        """Same call with raw host addresses (e.g. pinned buffers owned by the caller)."""
        self._check(self._lib.mascot_set_ratings(self._h, C.c_void_p(train_ptr), C.c_uint64(n_train), C.c_void_p(test_ptr),
                                                 C.c_uint64(n_test), C.c_uint32(n_users), C.c_uint32(n_items)))
        self.n_users, self.n_items, self.n_train, self.n_test = n_users, n_items, n_train, n_test

    # ---- sharded training building blocks ----
    def set_ratings_sharded(self, train, segment_offsets, test, n_users, n_items, user_degree=None, item_degree=None):
        train, test = as_ratings(train), as_ratings(test)
        seg = np.ascontiguousarray(segment_offsets, np.uint64)
        ud = None if user_degree is None else np.ascontiguousarray(user_degree, np.uint32)
        idg = None if item_degree is None else np.ascontiguousarray(item_degree, np.uint32)
        self._check(self._lib.mascot_set_ratings_sharded(self._h, _ptr(train), C.c_uint64(train.size), _ptr(seg), C.c_uint32(seg.size - 1),
                                                         _ptr(test), C.c_uint64(test.size), C.c_uint32(n_users), C.c_uint32(n_items),
                                                         _ptr(ud), _ptr(idg)))
        self.n_users, self.n_items, self.n_train, self.n_test = n_users, n_items, train.size, test.size

    def is_check_epoch(self, epoch):
        return bool(self._lib.mascot_is_check_epoch(self._h, C.c_uint32(epoch)))

    def stats_begin(self):
        self._check(self._lib.mascot_stats_begin(self._h))

    def train_segment(self, epoch, segment, collect_stats=False, wait=True):
        st = EpochStats() if wait else None
        self._check(self._lib.mascot_train_segment(self._h, C.c_uint32(epoch), C.c_uint32(segment), C.c_uint32(1 if collect_stats else 0),
                                                   C.byref(st) if wait else None))
        return st

    def stats_fetch(self):
        ug, ig = len(self.group_info(0)[0]), len(self.group_info(1)[0])
        out = [np.empty(ug * self.k, np.float32), np.empty(ig * self.k, np.float32), np.empty(ug, np.float32), np.empty(ig, np.float32)]
        self._check(self._lib.mascot_stats_fetch(self._h, *[_ptr(a) for a in out]))
        return out

    def stats_apply(self, epoch, gsum_p, gsum_q, nsum_p, nsum_q):
        arrs = [np.ascontiguousarray(a, np.float32) for a in (gsum_p, gsum_q, nsum_p, nsum_q)]
        pu, pi = C.c_uint32(), C.c_uint32()
        self._check(self._lib.mascot_stats_apply(self._h, C.c_uint32(epoch), *[_ptr(a) for a in arrs], C.byref(pu), C.byref(pi)))
        return pu.value, pi.value

    def item_rows(self, row_begin, row_end):
        p16, b16, p32, b32 = C.c_void_p(), C.c_uint64(), C.c_void_p(), C.c_uint64()
        self._check(self._lib.mascot_item_rows(self._h, C.c_uint32(row_begin), C.c_uint32(row_end), C.byref(p16), C.byref(b16),
                                               C.byref(p32), C.byref(b32)))
        return (p16.value or 0, b16.value), (p32.value or 0, b32.value)

    def sync(self):
        self._check(self._lib.mascot_sync(self._h))

    def stream_handle(self):
        """Address of the engine's cudaStream_t (for ordering a caller's own device work on it)."""
        st = C.c_void_p()
        self._check(self._lib.mascot_get_stream(self._h, C.byref(st)))
        return st.value or 0

    def eval_sq_error(self):
        s, n = C.c_double(), C.c_uint64()
        self._check(self._lib.mascot_eval_sq_error(self._h, C.byref(s), C.byref(n)))
        return s.value, n.value

    def reload_train_raw(self, train_ptr, n_train):
        """Replace the training stream from a raw host address (the per-step input path)."""
        self._check(self._lib.mascot_reload_train(self._h, C.c_void_p(train_ptr), C.c_uint64(n_train)))
        self.n_train = n_train

    def train_epoch_streamed_raw(self, epoch, train_ptr, n_train):
        """One epoch over a rating array in host memory (upload overlapped with the updates)."""
        st = EpochStats()
        self._check(self._lib.mascot_train_epoch_streamed(self._h, C.c_uint32(epoch), C.c_void_p(train_ptr), C.c_uint64(n_train), C.byref(st)))
        self.n_train = n_train
        return st

    def train_epoch_streamed(self, epoch, train):
        train = as_ratings(train)
        return self.train_epoch_streamed_raw(epoch, train.ctypes.data, train.size)

    def reload_train(self, train):
        train = as_ratings(train)
        self.reload_train_raw(train.ctypes.data, train.size)

    # ---- sharded training inside the library (one engine per GPU, NCCL between them) ----
    def shard_init(self, comm_id, rank, world, blocks_per_gpu=1, timeout_ms=0):
        """Join the group identified by the 128 bytes `comm_id` (see comm_unique_id)."""
        buf = (C.c_ubyte * COMM_ID_BYTES).from_buffer_copy(bytes(comm_id))
        self._check(self._lib.mascot_shard_init(self._h, buf, C.c_uint32(rank), C.c_uint32(world), C.c_uint32(blocks_per_gpu),
                                                C.c_uint32(timeout_ms)))

    def shard_set_ratings(self, train, test, n_users, n_items):
        train, test = as_ratings(train), as_ratings(test)
        self.shard_set_ratings_raw(train.ctypes.data, train.size, test.ctypes.data, test.size, n_users, n_items)

    def shard_set_ratings_raw(self, train_ptr, n_train, test_ptr, n_test, n_users, n_items):
        self._check(self._lib.mascot_shard_set_ratings(self._h, C.c_void_p(train_ptr), C.c_uint64(n_train), C.c_void_p(test_ptr),
                                                       C.c_uint64(n_test), C.c_uint32(n_users), C.c_uint32(n_items)))
        info = self.shard_info()
        self.n_users, self.n_items, self.n_train, self.n_test = n_users, n_items, info["local_ratings"], info["local_test_ratings"]

    def shard_train_epoch(self, epoch):
        st = EpochStats()
        self._check(self._lib.mascot_shard_train_epoch(self._h, C.c_uint32(epoch), C.byref(st)))
        return st

    def shard_eval_rmse(self):
        v = C.c_double()
        self._check(self._lib.mascot_shard_eval_rmse(self._h, C.byref(v)))
        return v.value

    def shard_gather_factors(self):
        self._check(self._lib.mascot_shard_gather_factors(self._h))

    def shard_info(self):
        r, w, b, n, nt, sent = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        self._check(self._lib.mascot_shard_info(self._h, C.byref(r), C.byref(w), C.byref(b), C.byref(n), C.byref(nt), C.byref(sent)))
        return dict(rank=r.value, world=w.value, blocks=b.value, local_ratings=n.value, local_test_ratings=nt.value, bytes_sent=sent.value)

    def release_scratch(self):
        self._check(self._lib.mascot_release_scratch(self._h))

    def init_factors(self):
        self._check(self._lib.mascot_init_factors(self._h))

    def set_factors(self, P, Q):
        P = np.ascontiguousarray(P, np.float32)
        Q = np.ascontiguousarray(Q, np.float32)
        assert P.size == self.n_users * self.k and Q.size == self.n_items * self.k
        self._check(self._lib.mascot_set_factors(self._h, _ptr(P), _ptr(Q)))

    def train_epoch(self, epoch):
        st = EpochStats()
        self._check(self._lib.mascot_train_epoch(self._h, C.c_uint32(epoch), C.byref(st)))
        return st

    def eval_rmse(self):
        v = C.c_double()
        self._check(self._lib.mascot_eval_rmse(self._h, C.byref(v)))
        return v.value

    def get_factors(self, order=0):
        P = np.empty((self.n_users, self.k), np.float32)
        Q = np.empty((self.n_items, self.k), np.float32)
        self._check(self._lib.mascot_get_factors(self._h, _ptr(P), _ptr(Q), C.c_int(order)))
        return P, Q

    def group_info(self, side):
        n = C.c_uint32()
        self._check(self._lib.mascot_get_group_info(self._h, C.c_int(side), C.byref(n), None, None, None))
        end = np.empty(n.value, np.uint32)
        prec = np.empty(n.value, np.uint8)
        err = np.empty(n.value, np.float32)
        self._check(self._lib.mascot_get_group_info(self._h, C.c_int(side), C.byref(n), _ptr(end), _ptr(prec), _ptr(err)))
        return end, prec, err

    def promote_group(self, side, group):
        self._check(self._lib.mascot_promote_group(self._h, C.c_int(side), C.c_uint32(group)))

    def index_maps(self):
        u = np.empty(self.n_users, np.uint32)
        i = np.empty(self.n_items, np.uint32)
        self._check(self._lib.mascot_get_index_maps(self._h, _ptr(u), _ptr(i)))
        return u, i

    def sample_stats(self):
        ug, ig = len(self.group_info(0)[0]), len(self.group_info(1)[0])
        gp = np.empty(ug * self.k, np.float32)
        gq = np.empty(ig * self.k, np.float32)
        np_ = np.empty(ug, np.float32)
        nq = np.empty(ig, np.float32)
        self._check(self._lib.mascot_get_sample_stats(self._h, _ptr(gp), _ptr(gq), _ptr(np_), _ptr(nq)))
        return gp, gq, np_, nq

    def test_ratings(self, order=1):
        out = np.empty(self.n_test, RATING)
        self._check(self._lib.mascot_get_test_ratings(self._h, _ptr(out), C.c_int(order)))
        return out

    def stream_order(self):
        out = np.empty(self.n_train, np.uint32)
        self._check(self._lib.mascot_get_stream_order(self._h, _ptr(out)))
        return out

    def stream_source_index(self, pos):
        v = C.c_uint64()
        self._check(self._lib.mascot_stream_source_index(self._h, C.c_uint64(pos), C.byref(v)))
        return v.value


def write_binary_ratings(path, records, n_users, n_items):
    """Write the binary rating file of the command-line tools (cli/io_formats.h): `records` is an (n, 3)
    uint32 view or a RATING array with compact ids."""
    recs = as_ratings(records)
    header = np.zeros(1, np.dtype([("magic", "<u4"), ("version", "<u4"), ("n", "<u8"), ("n_users", "<u4"), ("n_items", "<u4"),
                                   ("flags", "<u4"), ("reserved", "<u4")]))
    header["magic"], header["version"], header["n"] = 0x5243534d, 1, recs.size
    header["n_users"], header["n_items"], header["flags"] = n_users, n_items, 1
    with open(path, "wb") as f:
        f.write(header.tobytes())
        recs.tofile(f)


def comm_unique_id():
    """128 opaque bytes naming a new group of sharded engines (made by one rank, carried to the others)."""
    buf = (C.c_ubyte * COMM_ID_BYTES)()
    rc = load().mascot_comm_unique_id(buf)
    if rc != OK:
        raise MascotError(rc, load().mascot_last_error(None).decode())
    return bytes(buf)


def shard_schedule(world, blocks_per_gpu, rank, step):
    """(block trained, rank it is sent to, block that arrives, rank it comes from) - needs no device."""
    out = [C.c_uint32() for _ in range(4)]
    rc = load().mascot_shard_schedule(C.c_uint32(world), C.c_uint32(blocks_per_gpu), C.c_uint32(rank), C.c_uint32(step),
                                      *[C.byref(o) for o in out])
    if rc != OK:
        raise MascotError(rc, "bad schedule arguments")
    return tuple(o.value for o in out)


def probe_read_bandwidth(nbytes, passes=20, device=0):
    """GB/s of 128-bit L2-only loads over a buffer of `nbytes` (L2-resident when small, HBM when large)."""
    v = C.c_double()
    rc = load().mascot_probe_read_bandwidth(C.c_int(device), C.c_uint64(nbytes), C.c_uint32(passes), C.byref(v))
    if rc != OK:
        raise MascotError(rc, load().mascot_last_error(None).decode())
    return v.value


def rmse_host(P, Q, test, k, device=0):
    """Handle-free evaluation of fp32 factors on host buffers (the test_mf path)."""
    L = load()
    P = np.ascontiguousarray(P, np.float32)
    Q = np.ascontiguousarray(Q, np.float32)
    test = as_ratings(test)
    v = C.c_double()
    rc = L.mascot_rmse_host(_ptr(P), C.c_uint32(P.size // k), _ptr(Q), C.c_uint32(Q.size // k), C.c_uint32(k),
                            _ptr(test), C.c_uint64(test.size), C.c_int(device), C.byref(v))
    if rc != OK:
        raise MascotError(rc, L.mascot_last_error(None).decode())
    return v.value
