"""ctypes binding of the CPU oracle (oracle/liboracle.so).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke test and the CPU-baseline leg of bench.py may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

NODE = np.dtype([("r", np.float32), ("u", np.uint32), ("i", np.uint32)])


class Rules(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("dot_f32", "inner_f32", "outer_f32", "chain_f32", "norm_f32",
                                       "dot_f16", "inner_f16", "mpt_outer", "stats_sum", "mup_fwd_f16", "mup_bwd_f16", "afp_avg")]

    def __repr__(self):
        return "Rules(" + ", ".join(f"{n}={getattr(self, n)}" for n, _ in self._fields_) + ")"


def build():
    """Compile liboracle.so with the committed Makefile (gcc, seconds)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.mo_h2f.restype = C.c_float
        L.mo_h2f.argtypes = [C.c_uint16]
        L.mo_f2h.restype = C.c_uint16
        L.mo_f2h.argtypes = [C.c_float]
        for f in ("mo_hadd", "mo_hsub", "mo_hmul"):
            getattr(L, f).restype = C.c_uint16
            getattr(L, f).argtypes = [C.c_uint16, C.c_uint16]
        L.mo_hfma.restype = C.c_uint16
        L.mo_hfma.argtypes = [C.c_uint16] * 3
        L.mo_rmse_literal.restype = C.c_float
        L.mo_rmse_double.restype = C.c_double
        L.mo_grouping.restype = C.c_int
        L.mo_is_check_epoch.restype = C.c_int
        L.mo_max_threads.restype = C.c_int
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def rules_literal():
    r = Rules()
    lib().mo_rules_literal(C.byref(r))
    return r


def rules_reference():
    r = Rules()
    lib().mo_rules_reference_build(C.byref(r))
    return r


def as_nodes(R):
    """Accept an (n,3) uint32 view or a NODE structured array; return a contiguous NODE array."""
    R = np.ascontiguousarray(R)
    if R.dtype == NODE:
        return R
    return R.reshape(-1, 3).astype(np.uint32, copy=False).view(NODE).reshape(-1)


def f2h(a):
    """float32 array -> binary16 bit patterns (uint16), round to nearest even (numpy does the same)."""
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def h2f(a):
    return np.asarray(a, np.uint16).view(np.float16).astype(np.float32)


def lr_schedule(alpha, decay, epochs):
    out = np.empty(epochs, np.float32)
    lib().mo_lr_schedule(C.c_float(alpha), C.c_float(decay), C.c_int(epochs), _p(out))
    return out


def init_normal(count, seed, sid):
    """Host twin of the engine's seeded factor initialisation (stream 1: users, 2: items)."""
    out = np.empty(int(count), np.float32)
    lib().mo_init_normal(_p(out), C.c_uint64(int(count)), C.c_uint64(int(seed)), C.c_uint64(int(sid)))
    return out


def is_check_epoch(e, epochs, interval):
    return bool(lib().mo_is_check_epoch(C.c_int(e), C.c_int(epochs), C.c_int(interval)))


def degree_sort(ids, n_entities):
    ids = np.ascontiguousarray(ids, np.uint32)
    s2o = np.empty(n_entities, np.uint32)
    o2s = np.empty(n_entities, np.uint32)
    cnt = np.empty(n_entities, np.uint32)
    lib().mo_degree_sort(_p(ids), C.c_uint64(ids.size), C.c_uint64(1), C.c_uint32(n_entities), _p(s2o), _p(o2s), _p(cnt))
    return s2o, o2s, cnt


def grouping(cnt_sorted, requested):
    cnt_sorted = np.ascontiguousarray(cnt_sorted, np.uint32)
    end = np.empty(cnt_sorted.size, np.uint32)
    gof = np.empty(cnt_sorted.size, np.uint32)
    g = lib().mo_grouping(_p(cnt_sorted), C.c_uint32(cnt_sorted.size), C.c_uint32(requested), _p(end), _p(gof))
    return end[:g].copy(), gof


def group_errors(grad_sum, norm_sum, k, prec, initial):
    groups = len(prec)
    grad_sum = np.ascontiguousarray(grad_sum, np.float32)
    norm_sum = np.ascontiguousarray(norm_sum, np.float32).reshape(groups, -1)
    prec = np.ascontiguousarray(prec, np.uint8)
    initial = np.ascontiguousarray(initial, np.float32)
    out = np.empty(groups, np.float32)
    lib().mo_group_errors(_p(grad_sum), _p(norm_sum), C.c_int(norm_sum.shape[1]), C.c_int(groups), C.c_int(k),
                          _p(prec), _p(initial), _p(out))
    return out


def _seq(seq):
    if seq is None:
        return None
    return np.ascontiguousarray(seq, np.uint32)


def sgd_run(k, R, seq, P, Q, lr, lam, rules, n=None):
    R = as_nodes(R)
    seq = _seq(seq)
    nseq = seq.size if seq is not None else (R.size if n is None else n)
    lib().mo_sgd_run(C.c_int(k), _p(R), _p(seq), C.c_uint64(nseq), _p(P), _p(Q), C.c_float(lr), C.c_float(lam), C.byref(rules))


def mpt_run(k, R, seq, P, Q, lr, lam, rules):
    R = as_nodes(R)
    seq = _seq(seq)
    nseq = seq.size if seq is not None else R.size
    lib().mo_mpt_run(C.c_int(k), _p(R), _p(seq), C.c_uint64(nseq), _p(P), _p(Q), C.c_float(lr), C.c_float(lam), C.byref(rules))


def muppet_run(k, R, seq, P, Q, lr, lam, bits_fwd, bits_bwd, rules, first_sample_pos=None):
    """Returns (sum_updated_val[k], sum_norms) of the sampled ratings; P, Q are updated in place."""
    R = as_nodes(R)
    seq = _seq(seq)
    nseq = seq.size if seq is not None else R.size
    fsp = nseq if first_sample_pos is None else first_sample_pos
    suv = np.zeros(k, np.float32)
    sn = np.zeros(1, np.float32)
    lib().mo_muppet_run(C.c_int(k), _p(R), _p(seq), C.c_uint64(nseq), _p(P), _p(Q), C.c_float(lr), C.c_float(lam),
                        C.c_int(bits_fwd), C.c_int(bits_bwd), C.c_uint64(fsp), _p(suv), _p(sn), C.byref(rules))
    return suv, float(sn[0])


def switching_run(k, R, seq, P, Q, precision, lr, lam, rules, first_sample_pos=None):
    """-v 8 trainer: P, Q are uint16 arrays (binary16 bit patterns) for precision 0, float32 for 1.
    Returns (sum_updated_val[k], sum_norms); P, Q are updated in place."""
    R = as_nodes(R)
    seq = _seq(seq)
    nseq = seq.size if seq is not None else R.size
    fsp = nseq if first_sample_pos is None else first_sample_pos
    suv = np.zeros(k, np.float32)
    sn = np.zeros(1, np.float32)
    lib().mo_switching_run(C.c_int(k), _p(R), _p(seq), C.c_uint64(nseq), _p(P), _p(Q), C.c_int(precision), C.c_float(lr),
                           C.c_float(lam), C.c_uint64(fsp), _p(suv), _p(sn), C.byref(rules))
    return suv, float(sn[0])


def afp_run(k, R, seq, P, Q, lr, lam, epoch, init_threshold, rules):
    R = as_nodes(R)
    seq = _seq(seq)
    nseq = seq.size if seq is not None else R.size
    lib().mo_afp_run(C.c_int(k), _p(R), _p(seq), C.c_uint64(nseq), _p(P), _p(Q), C.c_float(lr), C.c_float(lam),
                     C.c_int(epoch), C.c_int(init_threshold), C.byref(rules))


def memquant_run(k, R, seq, P16, Q16, lr, lam, rules):
    R = as_nodes(R)
    seq = _seq(seq)
    nseq = seq.size if seq is not None else R.size
    lib().mo_memquant_run(C.c_int(k), _p(R), _p(seq), C.c_uint64(nseq), _p(P16), _p(Q16), C.c_float(lr), C.c_float(lam), C.byref(rules))


class MascotModel:
    """Mixed-precision factor store in logical element order: every row lives either in the
    binary16 arrays (precision 0) or in the fp32 arrays (precision 1), chosen by its group."""

    def __init__(self, k, P, Q, ugroup, igroup, uprec, iprec):
        self.k = k
        self.ugroup = np.ascontiguousarray(ugroup, np.uint32)
        self.igroup = np.ascontiguousarray(igroup, np.uint32)
        self.uprec = np.ascontiguousarray(uprec, np.uint8).copy()
        self.iprec = np.ascontiguousarray(iprec, np.uint8).copy()
        P = np.ascontiguousarray(P, np.float32).reshape(-1, k)
        Q = np.ascontiguousarray(Q, np.float32).reshape(-1, k)
        self.P32, self.Q32 = P.copy(), Q.copy()
        self.P16, self.Q16 = f2h(P), f2h(Q)

    @property
    def uprec_row(self):
        return np.ascontiguousarray(self.uprec[self.ugroup])

    @property
    def iprec_row(self):
        return np.ascontiguousarray(self.iprec[self.igroup])

    def promote(self, side, g):
        """precision_switching.h:8-51: widen one group's rows to fp32, one way."""
        if side == "u":
            rows = self.ugroup == g
            self.P32[rows] = h2f(self.P16[rows])
            self.uprec[g] = 1
        else:
            rows = self.igroup == g
            self.Q32[rows] = h2f(self.Q16[rows])
            self.iprec[g] = 1

    def factors(self):
        P = np.where(self.uprec_row[:, None] == 1, self.P32, h2f(self.P16))
        Q = np.where(self.iprec_row[:, None] == 1, self.Q32, h2f(self.Q16))
        return P.astype(np.float32), Q.astype(np.float32)

    def run(self, R, seq, lr, lam, rules, first_sample_pos=None, stats=False, item_stats_by_run=False, into=None):
        """`into`: four existing statistic arrays to keep accumulating into (instead of fresh zeros)."""
        R = as_nodes(R)
        seq = _seq(seq)
        nseq = seq.size if seq is not None else R.size
        k = self.k
        ug, ig = len(self.uprec), len(self.iprec)
        if stats and into is not None:
            gp, gq, np_, nq = into
        elif stats:
            gp, gq = np.zeros(ug * k, np.float32), np.zeros(ig * k, np.float32)
            np_, nq = np.zeros(ug, np.float32), np.zeros(ig, np.float32)
        else:
            gp = gq = np_ = nq = None
        fsp = nseq if first_sample_pos is None else first_sample_pos
        upr, ipr = self.uprec_row, self.iprec_row
        lib().mo_mascot_run(C.c_int(k), _p(R), _p(seq), C.c_uint64(nseq),
                            _p(self.P16), _p(self.P32), _p(upr), _p(self.ugroup),
                            _p(self.Q16), _p(self.Q32), _p(ipr), _p(self.igroup),
                            C.c_float(lr), C.c_float(lam), C.c_uint64(fsp),
                            _p(gp), _p(gq), _p(np_), _p(nq), C.c_int(1 if item_stats_by_run else 0), C.byref(rules))
        return gp, gq, np_, nq


def rmse_literal(k, T, P, Q, rules):
    T = as_nodes(T)
    P = np.ascontiguousarray(P, np.float32)
    Q = np.ascontiguousarray(Q, np.float32)
    blocks = (T.size + 511) // 512
    be = np.zeros(max(blocks, 1), np.float32)
    v = lib().mo_rmse_literal(C.c_int(k), _p(T), C.c_uint32(T.size), _p(P), _p(Q), _p(be), C.byref(rules))
    return float(v), be[:blocks]


def rmse_double(k, T, P, Q):
    T = as_nodes(T)
    P = np.ascontiguousarray(P, np.float32)
    Q = np.ascontiguousarray(Q, np.float32)
    return float(lib().mo_rmse_double(C.c_int(k), _p(T), C.c_uint64(T.size), _p(P), _p(Q)))


def max_threads():
    return int(lib().mo_max_threads())


def sgd_epoch_hogwild(k, R, P, Q, lr, lam, threads, rules):
    R = as_nodes(R)
    lib().mo_sgd_epoch_hogwild(C.c_int(k), _p(R), C.c_uint64(R.size), _p(P), _p(Q), C.c_float(lr), C.c_float(lam),
                               C.c_int(threads), C.byref(rules))


def mascot_epoch_hogwild(model, R, lr, lam, threads, rules):
    R = as_nodes(R)
    upr, ipr = model.uprec_row, model.iprec_row
    lib().mo_mascot_epoch_hogwild(C.c_int(model.k), _p(R), C.c_uint64(R.size),
                                  _p(model.P16), _p(model.P32), _p(upr), _p(model.Q16), _p(model.Q32), _p(ipr),
                                  C.c_float(lr), C.c_float(lam), C.c_int(threads), C.byref(rules))


# ---- the fast host-core baseline (oracle/host_loop.cpp): measured by bench.py, checked by RMSE only ----
_HL = None


def host_loop():
    """ctypes handle of libhostloop.so; raises when the CPU lacks AVX2 / F16C / FMA."""
    global _HL
    if _HL is None:
        path = os.path.join(_HERE, "libhostloop.so")
        if not os.path.exists(path):
            subprocess.check_call(["make", "-s", "-C", _HERE, "libhostloop.so"])
        L = C.CDLL(path)
        L.hl_max_threads.restype = C.c_int
        L.hl_supported.restype = C.c_int
        if not L.hl_supported():
            raise OSError("this CPU lacks AVX2 / F16C / FMA: the fast host loop cannot run here")
        _HL = L
    return _HL


class HostLoopModel:
    """Factors of the fast host loop: binary16 rows (MASCOT, all groups still binary16) or fp32 rows (SGD)."""

    def __init__(self, k, P, Q, half):
        self.k, self.half = int(k), bool(half)
        L = host_loop()
        P = np.ascontiguousarray(P, np.float32); Q = np.ascontiguousarray(Q, np.float32)
        if half:
            self.P = np.empty(P.shape, np.uint16); self.Q = np.empty(Q.shape, np.uint16)
            L.hl_to_half(_p(P), _p(self.P), C.c_uint64(P.size)); L.hl_to_half(_p(Q), _p(self.Q), C.c_uint64(Q.size))
        else:
            self.P, self.Q = P.copy(), Q.copy()

    def epoch(self, R, lr, lam, threads):
        R = as_nodes(R)
        fn = host_loop().hl_mascot_half_epoch if self.half else host_loop().hl_sgd_epoch
        fn(C.c_int(self.k), _p(R), C.c_uint64(R.shape[0]), _p(self.P), _p(self.Q), C.c_float(lr), C.c_float(lam), C.c_int(threads))

    def factors(self):
        if not self.half:
            return self.P, self.Q
        P = np.empty(self.P.shape, np.float32); Q = np.empty(self.Q.shape, np.float32)
        host_loop().hl_to_float(_p(self.P), _p(P), C.c_uint64(P.size)); host_loop().hl_to_float(_p(self.Q), _p(Q), C.c_uint64(Q.size))
        return P, Q


def chunk_sequence(starts, vec, nnz):
    """Order in which one reference warp visits the rating array: for every drawn start, `vec`
    consecutive positions modulo nnz (sgd/sgd_kernel.h:21-33)."""
    starts = np.asarray(starts, np.uint64)
    return ((starts[:, None] + np.arange(vec, dtype=np.uint64)[None, :]) % np.uint64(nnz)).reshape(-1).astype(np.uint32)
