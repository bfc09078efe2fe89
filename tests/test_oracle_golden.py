"""CPU tests: the oracle against the golden vectors produced by the reference's own kernels
(tests/golden/harness_out.bin, generated on a B200 by oracle/ref_harness.cu from
tests/golden/harness_in.bin), and the oracle's primitives against independent restatements."""
import numpy as np
import pytest

from helpers import assert_bit_equal, golden_case, golden_mascot_model

KS = (128, 64)


@pytest.mark.parametrize("name", [f"sgd_k{k}{s}" for k in KS for s in ("", "_big", "_tight")])
def test_sgd_matches_reference_kernel(oracle, golden, name):
    I, G = golden
    c = golden_case(I, G, name, oracle)
    P, Q = c["P"].copy(), c["Q"].copy()
    oracle.sgd_run(c["k"], c["R"], c["seq"], P, Q, c["lr"], c["lam"], oracle.rules_reference())
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


def test_source_literal_rule_differs_from_the_built_reference(oracle, golden):
    """The unfused reading of the source is NOT what the compiled reference computes."""
    I, G = golden
    c = golden_case(I, G, "sgd_k128_big", oracle)
    P, Q = c["P"].copy(), c["Q"].copy()
    oracle.sgd_run(c["k"], c["R"], c["seq"], P, Q, c["lr"], c["lam"], oracle.rules_literal())
    assert (P.view(np.uint32) != G["sgd_k128_big.P_out"].reshape(P.shape).view(np.uint32)).any()


@pytest.mark.parametrize("name", [f"mascot_k{k}_{t}" for k in KS for t in ("mixed", "half", "float", "mixed_big")])
def test_mascot_matches_reference_kernel(oracle, golden, name):
    I, G = golden
    c = golden_case(I, G, name, oracle)
    m = golden_mascot_model(I, name, c, oracle)
    st = m.run(c["R"], c["seq"], c["lr"], c["lam"], oracle.rules_reference(), first_sample_pos=c["fs"], stats=True)
    P, Q = m.factors()
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")
    for got, key in zip(st, ("gsum_p", "gsum_q", "nsum_p", "nsum_q")):
        assert_bit_equal(got, G[f"{name}.{key}"], key)


@pytest.mark.parametrize("k", KS)
def test_mpt_matches_reference_kernel(oracle, golden, k):
    I, G = golden
    name = f"mpt_k{k}"
    c = golden_case(I, G, name, oracle)
    P, Q = c["P"].copy(), c["Q"].copy()
    oracle.mpt_run(c["k"], c["R"], c["seq"], P, Q, c["lr"], c["lam"], oracle.rules_reference())
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("name", [f"muppet_k{k}_b{b}" for k in KS for b in (8, 12, 14, 16, 32)])
def test_muppet_matches_reference_kernel(oracle, golden, name):
    """Factors and both sampled statistics of muppet_sgd_k128/k64_hogwild_kernel at every pass width."""
    I, G = golden
    c = golden_case(I, G, name, oracle)
    P, Q = c["P"].copy(), c["Q"].copy()
    bits = c["extra0"]
    suv, sn = oracle.muppet_run(c["k"], c["R"], c["seq"], P, Q, c["lr"], c["lam"], bits, bits, oracle.rules_reference(),
                                first_sample_pos=c["fs"])
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")
    assert_bit_equal(suv, G[name + ".sum_updated_val"], "sum_updated_val")
    assert_bit_equal(np.float32(sn), G[name + ".sum_norms"], "sum_norms")
    if bits == 32:
        assert sn == 0 and not suv.any(), "no statistics at full width (muppet_sgd_kernel.h:266)"


@pytest.mark.parametrize("name", ["switching_k128_half", "switching_k128_half_big", "switching_k128_float"])
def test_switching_only_trainer_matches_reference_kernel(oracle, golden, name):
    """switching_only_sgd_k128_hogwild_kernel (-v 8) before (binary16 rows, statistics) and after its switch."""
    I, G = golden
    c = golden_case(I, G, name, oracle)
    precision = c["extra0"]
    if precision:
        P, Q = c["P"].copy(), c["Q"].copy()
    else:
        P, Q = oracle.f2h(c["P"]), oracle.f2h(c["Q"])
    suv, sn = oracle.switching_run(c["k"], c["R"], c["seq"], P, Q, precision, c["lr"], c["lam"], oracle.rules_reference(),
                                   first_sample_pos=c["fs"])
    if not precision:
        P, Q = oracle.h2f(P), oracle.h2f(Q)
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")
    assert_bit_equal(suv, G[name + ".sum_updated_val"], "sum_updated_val")
    assert_bit_equal(np.float32(sn), G[name + ".sum_norms"], "sum_norms")


@pytest.mark.parametrize("name", [f"mascot_k128_{t}" for t in ("mixed", "half", "float", "mixed_big")])
def test_naive_variant_equals_the_mascot_kernel(golden, name):
    """naive_mascot_sgd_k128_hogwild_kernel (-v 6) on the same inputs and random sequence as the MASCOT
    kernel: identical factors and statistics, i.e. it differs only in its group lookup."""
    _I, G = golden
    for key in ("P_out", "Q_out", "gsum_p", "gsum_q", "nsum_p", "nsum_q"):
        assert_bit_equal(G[f"{name}.naive_{key}"], G[f"{name}.{key}"], key)


@pytest.mark.parametrize("name", [f"afp_k{k}_e{e}" for k in KS for e in (0, 1)])
def test_afp_matches_reference_kernel(oracle, golden, name):
    """afp_sgd_k128/k64_hogwild_kernel in its first epoch (formats re-estimated at every rating for the
    first tenth) and in a later one (re-estimation intervals from QPA)."""
    I, G = golden
    c = golden_case(I, G, name, oracle)
    P, Q = c["P"].copy(), c["Q"].copy()
    threshold = int(np.float32(c["uc"] * c["vec"]) / np.float32(10.0))          # afp_sgd_kernel.h:143
    oracle.afp_run(c["k"], c["R"], c["seq"], P, Q, c["lr"], c["lam"], c["extra0"], threshold, oracle.rules_reference())
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("name", [f"memquant_k{k}{s}" for k in KS for s in ("", "_tight")])
def test_fp16_storage_trainer_matches_reference_kernel(oracle, golden, name):
    I, G = golden
    c = golden_case(I, G, name, oracle)
    P, Q = oracle.f2h(c["P"]), oracle.f2h(c["Q"])
    oracle.memquant_run(c["k"], c["R"], c["seq"], P, Q, c["lr"], c["lam"], oracle.rules_reference())
    assert_bit_equal(oracle.h2f(P), G[name + ".P_out"], "P")
    assert_bit_equal(oracle.h2f(Q), G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("name", [f"rmse_k{k}{s}" for k in KS for s in ("", "_tight")])
def test_rmse_matches_reference_kernel(oracle, golden, name):
    I, G = golden
    c = golden_case(I, G, name, oracle)
    v, blocks = oracle.rmse_literal(c["k"], c["R"], c["P"], c["Q"], oracle.rules_reference())
    assert_bit_equal(blocks, G[name + ".group_err"], "block partials")
    assert_bit_equal(np.float32(v), G[name + ".rmse"], "rmse")
    assert abs(v - oracle.rmse_double(c["k"], c["R"], c["P"], c["Q"])) <= 1e-3 * v


# ---- primitives ----------------------------------------------------------------------------

def test_half_conversion_every_bit_pattern(oracle):
    L = oracle.lib()
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([L.mo_h2f(int(x)) for x in h], np.float32)
    finite = ~np.isnan(want)
    assert (got[finite].view(np.uint32) == want[finite].view(np.uint32)).all()
    back = np.array([L.mo_f2h(float(x)) for x in want[finite]], np.uint16)
    assert (back == h[finite]).all()


def test_float_to_half_rounding_matches_numpy(oracle):
    L = oracle.lib()
    rng = np.random.default_rng(5)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 5, 20000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, 1e10, -1e10], np.float32),
    ])
    want = x.astype(np.float16).view(np.uint16)
    got = np.array([L.mo_f2h(float(v)) for v in x], np.uint16)
    assert (got == want).all()


def test_half_arithmetic_against_float16_and_exact_fma(oracle):
    from fractions import Fraction
    L = oracle.lib()
    rng = np.random.default_rng(6)
    a = (rng.standard_normal(3000) * 4).astype(np.float16)
    b = (rng.standard_normal(3000) * 0.3).astype(np.float16)
    c = (rng.standard_normal(3000) * 2).astype(np.float16)
    au, bu, cu = a.view(np.uint16), b.view(np.uint16), c.view(np.uint16)
    f32 = np.float32
    for j in range(a.size):
        x, y, z = int(au[j]), int(bu[j]), int(cu[j])
        assert L.mo_hadd(x, y) == np.float16(f32(a[j]) + f32(b[j])).view(np.uint16)
        assert L.mo_hmul(x, y) == np.float16(f32(a[j]) * f32(b[j])).view(np.uint16)
        assert L.mo_hsub(x, y) == np.float16(f32(a[j]) - f32(b[j])).view(np.uint16)
    # fma: exact rational arithmetic, then one rounding to binary16
    def round_half(fr):
        if fr == 0:
            return np.float16(0.0).view(np.uint16)
        # nearest-even on the exact value: compare against the two neighbouring halves
        approx = np.float16(float(fr))
        cands = {approx, np.nextafter(approx, np.float16(np.inf)), np.nextafter(approx, np.float16(-np.inf))}
        best = None
        for cand in cands:
            if not np.isfinite(cand):
                continue
            d = abs(Fraction(float(cand)) - fr)
            key = (d, int(cand.view(np.uint16)) & 1)
            if best is None or key < best[0]:
                best = (key, cand)
        return best[1].view(np.uint16)
    for j in range(1500):
        exact = Fraction(float(a[j])) * Fraction(float(b[j])) + Fraction(float(c[j]))
        assert L.mo_hfma(int(au[j]), int(bu[j]), int(cu[j])) == round_half(exact), j
    # a tie that only the exact product can break: 1.0 + (2^-11 + 2^-21) vs 1.0 + 2^-11
    one = np.float16(1.0).view(np.uint16)
    x = np.float16(2.0 ** -5).view(np.uint16)
    y = np.float16(2.0 ** -6 * (1 + 2.0 ** -10)).view(np.uint16)
    got = L.mo_hfma(int(x), int(y), int(one))
    assert got == np.float16(1.0 + 2.0 ** -10).view(np.uint16)


def test_lr_schedule_and_check_epochs(oracle):
    lr = oracle.lr_schedule(0.01, 0.1, 50)
    want = np.array([0.01 / (1.0 + np.float32(0.1).astype(np.float64) * e ** 1.5) for e in range(50)]).astype(np.float32)
    # alpha is a float in the reference too
    want = np.array([np.float64(np.float32(0.01)) / (1.0 + np.float64(np.float32(0.1)) * e ** 1.5) for e in range(50)]).astype(np.float32)
    assert (lr.view(np.uint32) == want.view(np.uint32)).all()
    checks = [e for e in range(50) if oracle.is_check_epoch(e, 50, 2)]
    assert checks == list(range(5, 49, 2))
    assert [e for e in range(8) if oracle.is_check_epoch(e, 8, 1)] == [5, 6]
    assert not any(oracle.is_check_epoch(e, 5, 1) for e in range(5))


def _grouping_bruteforce(cnt_sorted, requested):
    """Literal restatement of the reference's walk over degree classes."""
    n = len(cnt_sorted)
    threshold = int(np.ceil(np.float32(n) / np.float32(requested)))
    maxc = int(cnt_sorted[-1])
    last = {}
    for pos, c in enumerate(cnt_sorted):
        last[int(c)] = pos
    end, acc, prev = [], 0, 0
    for c in range(1, maxc + 1):
        if c in last:
            acc += last[c] - prev + 1
            if acc >= threshold:
                end.append(last[c]); acc = 0
            elif c == maxc:
                end.append(last[c])
            prev = last[c] + 1
    return end


@pytest.mark.parametrize("seed,n,req", [(0, 1000, 10), (1, 5000, 100), (2, 37, 5), (3, 64, 64), (4, 300, 1), (5, 2000, 500)])
def test_degree_sort_and_grouping(oracle, seed, n, req):
    rng = np.random.default_rng(seed)
    w = np.arange(1, n + 1, dtype=np.float64) ** -1.0
    ids = rng.choice(n, size=20 * n, p=w / w.sum()).astype(np.uint32)
    ids = np.concatenate([ids, np.arange(n, dtype=np.uint32)])      # every entity rated at least once
    s2o, o2s, cnt = oracle.degree_sort(ids, n)
    deg = np.bincount(ids, minlength=n)
    assert (np.diff(cnt.astype(np.int64)) >= 0).all()
    assert (deg[s2o] == cnt).all()
    assert (o2s[s2o] == np.arange(n)).all()
    same = cnt[1:] == cnt[:-1]
    assert (s2o[1:][same] > s2o[:-1][same]).all(), "ties keep ascending id order"
    end, gof = oracle.grouping(cnt, req)
    assert list(end) == _grouping_bruteforce(cnt, req)
    assert end[-1] == n - 1 and (np.diff(end.astype(np.int64)) > 0).all()
    for g, e in enumerate(end[:-1]):
        assert cnt[e] != cnt[e + 1], "a degree class is never split"
    assert (gof == np.searchsorted(end, np.arange(n), side="left")).all()


SETUP_CASES = ["setup_tiny_k128", "setup_zipf_k64", "setup_unrated_k128", "setup_flat_k64", "setup_manygroups_k128"]


@pytest.mark.parametrize("name", SETUP_CASES)
def test_setup_matches_reference_setup_functions(oracle, setup_golden, name):
    """Degree sort, grouping and index maps of the oracle against the tables the reference's own
    user_item_rating_histogram / split_group_based_equal_size_not_strict_ret_end_idx /
    matrix_reconstruction produced for the same ratings (tests/golden/setup_out.bin), including the
    order of entities with equal degree, unrated entities and a single degree class."""
    I, G = setup_golden
    meta = I[name + ".meta"]
    nu, ni, ug_req, ig_req = int(meta[2]), int(meta[3]), int(meta[6]), int(meta[7])
    R = I[name + ".R"].reshape(-1, 3)
    for side, col, n, req in (("user", 1, nu, ug_req), ("item", 2, ni, ig_req)):
        s2o, o2s, cnt = oracle.degree_sort(R[:, col], n)
        assert np.array_equal(cnt, G[f"{name}.{side}2cnt"]), "sorted degrees"
        assert np.array_equal(s2o, G[f"{name}.{side}2idx"]), "sorted position -> id (ties in ascending id order)"
        assert np.array_equal(o2s, G[f"{name}.{side}2sorted"]), "id -> sorted position"
        end, gof = oracle.grouping(cnt, req)
        assert np.array_equal(end, G[f"{name}.{'u' if side == 'user' else 'i'}end"]), "group end indices"
        assert np.array_equal(gof[o2s], G[f"{name}.{side}_group_idx"]), "group of every id"
        sizes = np.diff(np.concatenate([[-1], end.astype(np.int64)]))
        assert np.array_equal(sizes, G[f"{name}.{side}_group_size"])
    # the remapped rating arrays of matrix_reconst_gpu_triplet
    _, u2s, _ = oracle.degree_sort(R[:, 1], nu)
    _, i2s, _ = oracle.degree_sort(R[:, 2], ni)
    for key, src in (("R_sorted_ids", R), ("T_sorted_ids", I[name + ".T"].reshape(-1, 3))):
        want = G[f"{name}.{key}"].reshape(-1, 3)
        assert np.array_equal(src[:, 0], want[:, 0])
        assert np.array_equal(u2s[src[:, 1]], want[:, 1]) and np.array_equal(i2s[src[:, 2]], want[:, 2])
    # the scattered binary16 arenas: row of id e at its sorted position, rounded to nearest even
    k = int(meta[1])
    for key, src, o2s_ in (("P_arena", I[name + ".P"].reshape(nu, k), u2s), ("Q_arena", I[name + ".Q"].reshape(ni, k), i2s)):
        want = G[f"{name}.{key}"].reshape(-1, k)
        got = np.empty_like(src)
        got[o2s_] = oracle.h2f(oracle.f2h(src))
        assert_bit_equal(got, want, key)


def test_group_error_formula(oracle):
    rng = np.random.default_rng(9)
    k, groups = 64, 7
    gs = rng.standard_normal(groups * k).astype(np.float32)
    ns = (rng.random(groups).astype(np.float32) + 0.5) * 100
    prec = np.array([0, 1, 0, 0, 1, 0, 0], np.uint8)
    init = (rng.random(groups).astype(np.float32) + 0.5)
    got = oracle.group_errors(gs, ns, k, prec, init)
    for g in range(groups):
        if prec[g]:
            assert got[g] == -1
        else:
            num = np.float32(0)
            for d in range(k):
                num = np.float32(num + np.float32(gs[g * k + d]) ** 2)
            want = np.float32(np.float32(num / ns[g]) / init[g])
            assert abs(got[g] - want) <= 2e-6 * abs(want)
