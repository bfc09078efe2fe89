"""GPU tests of the engine's set-up path through the C ABI: the m-quantization tables against the
outputs of the reference's own set-up functions (tests/golden/setup_out.bin), the seeded factor
initialisation against its host twin in the oracle, the partition of the stream by precision class,
and the order of launches that once lost the shared-memory opt-in.  All comparisons are bit-exact
unless a tolerance is stated at the assertion."""
import numpy as np
import pytest

from helpers import assert_bit_equal, random_problem
from test_gpu_parity import make_engine, mascot_oracle_model
from test_oracle_golden import SETUP_CASES

pytestmark = pytest.mark.gpu


def _ratings(mascot, arr):
    return mascot.as_ratings(np.ascontiguousarray(arr.reshape(-1, 3)))


@pytest.mark.parametrize("name", SETUP_CASES)
def test_engine_setup_equals_reference_setup_functions(mascot, oracle, setup_golden, name):
    """mascot_set_ratings + mascot_set_factors of the MASCOT variant against user_item_rating_histogram,
    split_group_based_equal_size_not_strict_ret_end_idx, matrix_reconstruction (preprocess_utils.h:54-255)
    and cpy2grouped_parameters_gpu_for_comparison_indexing (model_init.cu:175-222) run by the harness."""
    I, G = setup_golden
    meta = I[name + ".meta"]
    k, nu, ni, ug_req, ig_req = int(meta[1]), int(meta[2]), int(meta[3]), int(meta[6]), int(meta[7])
    R, T = _ratings(mascot, I[name + ".R"]), _ratings(mascot, I[name + ".T"])
    P, Q = I[name + ".P"].reshape(nu, k), I[name + ".Q"].reshape(ni, k)
    for deterministic in (1, 0):
        eng = make_engine(mascot, mascot.V_MASCOT, k, deterministic=deterministic, shuffle=1 - deterministic,
                          user_group_num=ug_req, item_group_num=ig_req)
        eng.set_ratings(R, T, nu, ni)
        eng.set_factors(P, Q)
        u2s, i2s = eng.index_maps()
        assert np.array_equal(u2s, G[name + ".user2sorted"]) and np.array_equal(i2s, G[name + ".item2sorted"])
        assert np.array_equal(eng.group_info(0)[0], G[name + ".uend"])
        assert np.array_equal(eng.group_info(1)[0], G[name + ".iend"])
        Ps, Qs = eng.get_factors(1)
        assert_bit_equal(Ps, G[name + ".P_arena"], "binary16 user arena in sorted order")
        assert_bit_equal(Qs, G[name + ".Q_arena"], "binary16 item arena in sorted order")
        # the remapped test set: the same multiset of (r, sorted user, sorted item) records
        got = eng.test_ratings(1)
        want = _ratings(mascot, G[name + ".T_sorted_ids"])
        key = lambda a: np.lexsort((a["r"].view(np.uint32), a["i"], a["u"]))
        assert np.array_equal(got[key(got)], want[key(want)])
        # the training stream holds every remapped rating exactly once
        order = eng.stream_order()
        assert np.array_equal(np.sort(order), np.arange(R.size))
        eng.close()


@pytest.mark.parametrize("version,seed", [("sgd", 1), ("sgd", 0xfeedbeefcafe), ("mascot", 7), ("mpt", 3)])
def test_init_factors_equal_the_host_generator(mascot, oracle, version, seed):
    """mascot_init_factors against oracle.init_normal (stream 1: users, 2: items, caller's row order):
    fp32 variants bit for bit; binary16-stored rows equal the host values rounded to nearest even; MPT
    masters start from binary16 values (mf_methods.cu:730-733)."""
    k, nu, ni, n = 128, 1500, 900, 20000
    rng = np.random.default_rng(5)
    R, _, _ = random_problem(rng, nu, ni, n, k)
    vid = dict(sgd=mascot.V_SGD, mascot=mascot.V_MASCOT, mpt=mascot.V_MPT)[version]
    eng = make_engine(mascot, vid, k, seed=seed)
    eng.set_ratings(R, R[:10], nu, ni)
    eng.init_factors()
    P, Q = eng.get_factors(0)
    eng.close()
    Po = oracle.init_normal(nu * k, seed, 1).reshape(nu, k)
    Qo = oracle.init_normal(ni * k, seed, 2).reshape(ni, k)
    if version != "sgd":
        Po, Qo = oracle.h2f(oracle.f2h(Po)), oracle.h2f(oracle.f2h(Qo))
    assert_bit_equal(P, Po, "P"); assert_bit_equal(Q, Qo, "Q")
    assert abs(float(Po.std()) - 0.01) < 3e-4 and abs(float(Po.mean())) < 1e-4


@pytest.mark.parametrize("k", (128, 64))
def test_partitioned_stream_on_conflict_free_ratings_bit_exact(mascot, oracle, k):
    """Several workers + promoted groups: the stream is partitioned by precision class and every class
    runs its own kernel instantiation.  No two ratings share a user or an item, so the result does
    not depend on the order and must equal the sequential oracle bit for bit (plain stores).  Degree
    tables are given, so that the sides have several groups although every entity occurs once."""
    rng = np.random.default_rng(31 + k)
    n = 30011
    R = np.empty(n, mascot.RATING)
    R["u"] = rng.permutation(n); R["i"] = rng.permutation(n)
    R["r"] = rng.choice(np.arange(1, 6), n)
    P = (rng.standard_normal((n, k)) * 0.2).astype(np.float32)
    Q = (rng.standard_normal((n, k)) * 0.2).astype(np.float32)
    udeg = rng.integers(1, 40, n).astype(np.uint32)
    ideg = rng.integers(1, 40, n).astype(np.uint32)
    eng = make_engine(mascot, mascot.V_MASCOT, k, deterministic=0, shuffle=1, seed=17, user_group_num=8, item_group_num=8,
                      plain_user_stores=1, num_workers=700, sample_ratio=0.25, interval=1, error_threshold=1e9)
    seg = np.array([0, n // 3, n], np.uint64)               # two segments: classes are kept inside each
    eng.set_ratings_sharded(R, seg, R[:100], n, n, udeg, ideg)
    eng.set_factors(P, Q)
    model, u2s, i2s = mascot_oracle_model(oracle, eng, k, P, Q)
    assert len(eng.group_info(0)[0]) >= 4 and len(eng.group_info(1)[0]) >= 4
    for side, g in ((0, 1), (0, 3), (1, 0), (1, 2)):
        eng.promote_group(side, g); model.promote("u" if side == 0 else "i", g)
    order = eng.stream_order()
    assert np.array_equal(np.sort(order), np.arange(n)), "still every rating exactly once"
    # inside each segment the classes are contiguous, in the order hh, hf, fh, ff
    up, ip = model.uprec_row[u2s[R["u"][order]]], model.iprec_row[i2s[R["i"][order]]]
    cls = 2 * (up != 0) + (ip != 0)
    assert (np.isin(order[:n // 3], np.arange(n // 3))).all(), "segments keep their ratings"
    for lo, hi in ((0, n // 3), (n // 3, n)):
        assert (np.diff(cls[lo:hi].astype(np.int64)) >= 0).all()
        assert len(set(cls[lo:hi].tolist())) == 4
    rules = oracle.rules_reference()
    Rs = R.copy(); Rs["u"] = u2s[R["u"]]; Rs["i"] = i2s[R["i"]]
    lrs = oracle.lr_schedule(0.01, 0.1, 8)
    for e in range(7):                                       # epochs 5 and 6 are check epochs (statistics launches)
        st = eng.train_epoch(e)
        assert st.updates == n and st.error_check == (1 if e >= 5 else 0)
        model.run(Rs, None, float(lrs[e]), 0.05, rules)
    Po, Qo = model.factors()
    Pg, Qg = eng.get_factors(1)
    assert_bit_equal(Pg, Po, "P"); assert_bit_equal(Qg, Qo, "Q")
    # the sampled statistics: every launched range contributes its last quarter; compare against a
    # float64 recomputation over exactly those ratings (float32 sums in another order: 1e-4 relative)
    gp, gq, nsp, nsq = eng.sample_stats()
    assert np.isfinite(gp).all() and np.isfinite(nsq).all() and (nsp >= 0).all()
    assert (nsp[[1, 3]] == 0).all() and (nsq[[0, 2]] == 0).all(), "fp32 groups collect nothing"
    assert (np.delete(nsp, [1, 3]) > 0).all() and (np.delete(nsq, [0, 2]) > 0).all()
    eng.close()


def test_full_grid_then_single_block_then_full_grid(mascot):
    """One fp32 k=128 instantiation launched with a full grid, then by a deterministic engine (one
    small block), then with a full grid again in the same process: the second full-grid launch needs
    more dynamic shared memory than the default limit and must still succeed."""
    k, nu, ni, n = 128, 4000, 3000, 400000
    rng = np.random.default_rng(8)
    R, P, Q = random_problem(rng, nu, ni, n, k)
    rm = []
    for deterministic in (0, 1, 0):
        eng = make_engine(mascot, mascot.V_SGD, k, deterministic=deterministic, shuffle=1, num_workers=0 if deterministic else 2368)
        eng.set_ratings(R[:20000] if deterministic else R, R[:2000], nu, ni)
        eng.set_factors(P, Q)
        st = eng.train_epoch(0)
        assert st.workers == (1 if deterministic else st.workers) and (deterministic or st.workers >= 2368)
        rm.append(eng.eval_rmse())
        eng.close()
    assert all(np.isfinite(rm))


def test_ids_out_of_range_are_reported_and_never_used_as_an_index(mascot):
    """mascot_set_ratings, mascot_reload_train and mascot_train_epoch_streamed check ids on the device: a bad id
    gives MASCOT_ERR_BAD_ARG (the rating is replaced by a zero rating of row 0, no out-of-bounds access), and the
    engine keeps working once a valid array is loaded."""
    k, nu, ni, n = 64, 500, 400, 20000
    rng = np.random.default_rng(12)
    R, P, Q = random_problem(rng, nu, ni, n, k)
    bad = R.copy(); bad["u"][n // 2] = nu + 7
    bad_item = R.copy(); bad_item["i"][17] = 0x3fffffff
    eng = make_engine(mascot, mascot.V_SGD, k, deterministic=0, shuffle=1, num_workers=64)
    with pytest.raises(mascot.MascotError) as err:
        eng.set_ratings(bad, R[:100], nu, ni)
    assert err.value.status == mascot.ERR_BAD_ARG and "out of range" in str(err.value)
    with pytest.raises(mascot.MascotError) as err:
        eng.set_ratings(R, bad_item[:100], nu, ni)
    assert err.value.status == mascot.ERR_BAD_ARG
    eng.set_ratings(R, R[:100], nu, ni)
    eng.set_factors(P, Q)
    for broken in (bad, bad_item):
        with pytest.raises(mascot.MascotError) as err:
            eng.reload_train(broken)
        assert err.value.status == mascot.ERR_BAD_ARG
        with pytest.raises(mascot.MascotError) as err:
            eng.train_epoch_streamed(0, broken)
        assert err.value.status == mascot.ERR_BAD_ARG
    eng.reload_train(R)
    r0 = eng.eval_rmse()
    for e in range(3):
        eng.train_epoch(e)
    assert np.isfinite(eng.eval_rmse()) and eng.eval_rmse() < r0
    eng.close()


@pytest.mark.parametrize("window_log2,sorted_inside", [(0, True), (13, True), (12, False)])
def test_resident_stream_is_sorted_by_item_inside_run_windows(mascot, window_log2, sorted_inside):
    """Several workers, seeded permutation: the resident stream holds every rating exactly once and, inside
    windows of 2^13 positions, in ascending order of the item's arena row (mascot_config.run_window_log2:
    0 = automatic - 2^20 shortened to what 64 workers hold at one time, 64 x 8 chunks x 16 ratings = 2^13 -,
    13 = asked for, 12 = only the encoding step's windows of 4096 positions, which the check must notice)."""
    rng = np.random.default_rng(5)
    nu, ni, n = 3000, 700, 100_000
    R = np.empty(n, mascot.RATING)
    R["u"] = rng.integers(0, nu, n); R["i"] = rng.zipf(1.3, n) % ni
    R["r"] = rng.choice(np.arange(1, 6), n)
    eng = make_engine(mascot, mascot.V_SGD, 128, deterministic=0, shuffle=1, seed=3, num_workers=64, run_window_log2=window_log2)
    eng.set_ratings(R, R[:50], nu, ni)
    order = eng.stream_order()
    assert np.array_equal(np.sort(order), np.arange(n)), "every rating exactly once"
    _, i2s = eng.index_maps()
    rows = i2s[R["i"][order]].astype(np.int64)
    inside = np.ones(n - 1, bool)
    inside[np.arange(1, n) % 8192 == 0] = False                   # steps across a window boundary do not count
    ascending = bool((np.diff(rows)[inside] >= 0).all())
    assert ascending == sorted_inside
    # the encoding step's own windows are sorted in every case
    inside4k = np.ones(n - 1, bool); inside4k[np.arange(1, n) % 4096 == 0] = False
    assert (np.diff(rows)[inside4k] >= 0).all()
    # and the order is a permutation of the caller's, not the caller's own
    assert not np.array_equal(order, np.arange(n))
    P = (rng.standard_normal((nu, 128)) * 0.1).astype(np.float32); Q = (rng.standard_normal((ni, 128)) * 0.1).astype(np.float32)
    eng.set_factors(P, Q)
    before = eng.eval_rmse()
    for e in range(3):
        assert eng.train_epoch(e).updates == n
    assert eng.eval_rmse() < before
    eng.close()


def test_very_popular_users_train_with_thinned_reductions(mascot):
    """Three users own 45 % of the ratings; with 700 workers far more than 32 of them hold such a row at any
    time, so the engine marks those users and writes back only every 2^s-th of their updates (as reductions).
    The run must stay finite, learn (test RMSE falls), and end no worse than 5 % above the same run with plain
    stores for every user (mascot_config.plain_user_stores = 1), which is the reference's behaviour."""
    rng = np.random.default_rng(11)
    nu, ni, n, k = 4000, 3000, 600_000, 128
    Pt = rng.standard_normal((nu, 8)) * 0.5; Qt = rng.standard_normal((ni, 8)) * 0.5
    u = rng.integers(3, nu, n); hot = rng.random(n) < 0.45
    u[hot] = rng.integers(0, 3, hot.sum())
    i = rng.integers(0, ni, n)
    r = np.clip(np.rint(3.0 + (Pt[u] * Qt[i]).sum(1) + rng.standard_normal(n) * 0.3), 1, 5)
    R = mascot.make_ratings(u, i, r.astype(np.float32))
    train, test = R[: n - 20_000], R[n - 20_000:]
    P0 = (rng.standard_normal((nu, k)) * 0.05).astype(np.float32); Q0 = (rng.standard_normal((ni, k)) * 0.05).astype(np.float32)
    final = {}
    for plain in (0, 1):
        eng = make_engine(mascot, mascot.V_MASCOT, k, deterministic=0, shuffle=1, seed=9, num_workers=700, plain_user_stores=plain,
                          user_group_num=10, item_group_num=10, sample_ratio=0.05, interval=2, error_threshold=1e9, lam=0.02)
        eng.set_ratings(train, test, nu, ni)
        eng.set_factors(P0, Q0)
        before = eng.eval_rmse()
        for e in range(8):
            eng.train_epoch(e)
        final[plain] = eng.eval_rmse()
        Pg, Qg = eng.get_factors(1)
        assert np.isfinite(Pg).all() and np.isfinite(Qg).all()
        assert final[plain] < 0.9 * before, (before, final[plain])
        eng.close()
    assert final[0] <= 1.05 * final[1], final
