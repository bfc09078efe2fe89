"""GPU parity tests: libmascot, called through its C ABI, against the CPU oracle on the same seeded
inputs.  Integer work and every factor value are compared BIT-EXACTLY; the only floating-point
tolerance in this file is the comparison of the RMSE against a float64 recomputation (1e-5
relative, stated where it is used)."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_bit_equal, golden_case, random_problem, sort_like_reference

pytestmark = pytest.mark.gpu
KS = (128, 64)


def make_engine(mascot, version, k, **kw):
    base = dict(version=version, k=k, deterministic=1, shuffle=0, epoch=50, learning_rate=0.01, decay=0.1, lam=0.05)
    base.update(kw)
    return mascot.Engine(mascot.default_config(**base))


# --------------------------------------------------------------------------------------------
# golden vectors of the reference kernels, replayed through the engine
# --------------------------------------------------------------------------------------------
def replay_through_engine(mascot, version, c, half_inputs=False):
    """Feed the exact update sequence of a golden case as the training stream of a deterministic
    engine; epoch 0 of the schedule uses lr = alpha, so alpha is set to the case's lr."""
    seq = c["seq"]
    train = mascot.as_ratings(np.ascontiguousarray(c["R"][seq]))
    eng = make_engine(mascot, version, c["k"], learning_rate=c["lr"], lam=c["lam"])
    test = train[:1]
    eng.set_ratings(train, test, c["nu"], c["ni"])
    eng.set_factors(c["P"], c["Q"])
    st = eng.train_epoch(0)
    assert st.updates == len(seq) and np.float32(st.lr) == np.float32(c["lr"])
    P, Q = eng.get_factors(0)
    eng.close()
    return P, Q


@pytest.mark.parametrize("name", [f"sgd_k{k}{s}" for k in KS for s in ("", "_big", "_tight")])
def test_golden_fp32_sgd(mascot, oracle, golden, name):
    I, G = golden
    c = golden_case(I, G, name, oracle)
    P, Q = replay_through_engine(mascot, mascot.V_SGD, c)
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("k", KS)
def test_golden_mpt(mascot, oracle, golden, k):
    I, G = golden
    name = f"mpt_k{k}"
    c = golden_case(I, G, name, oracle)
    P, Q = replay_through_engine(mascot, mascot.V_MPT, c)
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("name", [f"memquant_k{k}{s}" for k in KS for s in ("", "_tight")])
def test_golden_fp16_storage(mascot, oracle, golden, name):
    I, G = golden
    c = golden_case(I, G, name, oracle)
    P, Q = replay_through_engine(mascot, mascot.V_MEMQUANT, c)
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("name", [f"mascot_k{k}_{t}" for k in KS for t in ("half", "float")])
def test_golden_mascot_uniform_precision(mascot, oracle, golden, name):
    """All-fp16 golden cases run as a fresh MASCOT engine (every group starts in fp16).  The all-fp32
    MASCOT case compiles to the same operations as the plain fp32 trainer, so it is replayed through
    the fp32 SGD engine - which also pins that equivalence."""
    I, G = golden
    c = golden_case(I, G, name, oracle)
    if name.endswith("float"):
        P, Q = replay_through_engine(mascot, mascot.V_SGD, c)
    else:
        seq = c["seq"]
        train = mascot.as_ratings(np.ascontiguousarray(c["R"][seq]))
        eng = make_engine(mascot, mascot.V_MASCOT, c["k"], learning_rate=c["lr"], lam=c["lam"], user_group_num=3, item_group_num=3)
        eng.set_ratings(train, train[:1], c["nu"], c["ni"])
        eng.set_factors(c["P"], c["Q"])
        eng.train_epoch(0)
        P, Q = eng.get_factors(0)
        eng.close()
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("name", [f"rmse_k{k}{s}" for k in KS for s in ("", "_tight")])
def test_golden_rmse_handle_free(mascot, oracle, golden, name):
    I, G = golden
    c = golden_case(I, G, name, oracle)
    v = mascot.rmse_host(c["P"], c["Q"], c["R"], c["k"])
    assert_bit_equal(np.float32(v), G[name + ".rmse"], "rmse")


# --------------------------------------------------------------------------------------------
# seeded problems: deterministic engine vs sequential oracle
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("k", KS)
@pytest.mark.parametrize("version", ["sgd", "mpt", "memquant"])
def test_deterministic_epochs_bit_exact(mascot, oracle, k, version):
    rng = np.random.default_rng(100 + k)
    n_users, n_items, n = 211, 157, 4999          # ragged: not a multiple of the chunk size
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=0.2)
    test = R[:700]
    vid = dict(sgd=mascot.V_SGD, mpt=mascot.V_MPT, memquant=mascot.V_MEMQUANT)[version]
    eng = make_engine(mascot, vid, k)
    eng.set_ratings(R, test, n_users, n_items)
    eng.set_factors(P, Q)
    lrs = oracle.lr_schedule(0.01, 0.1, 50)
    rules = oracle.rules_reference()
    if version == "memquant":
        P16, Q16 = oracle.f2h(P), oracle.f2h(Q)
    elif version == "mpt":
        Po, Qo = oracle.h2f(oracle.f2h(P)), oracle.h2f(oracle.f2h(Q))   # masters start from fp16 values
    else:
        Po, Qo = P.copy(), Q.copy()
    for e in range(3):
        st = eng.train_epoch(e)
        assert st.updates == n and st.kernel_launches == 1
        assert_bit_equal(np.float32(st.lr), lrs[e], "lr")
        if version == "sgd":
            oracle.sgd_run(k, R, None, Po, Qo, float(lrs[e]), 0.05, rules)
        elif version == "mpt":
            oracle.mpt_run(k, R, None, Po, Qo, float(lrs[e]), 0.05, rules)
        else:
            oracle.memquant_run(k, R, None, P16, Q16, float(lrs[e]), 0.05, rules)
    Pg, Qg = eng.get_factors(0)
    if version == "memquant":
        Po, Qo = oracle.h2f(P16), oracle.h2f(Q16)
    assert_bit_equal(Pg, Po, "P")
    assert_bit_equal(Qg, Qo, "Q")
    # test RMSE, reduced exactly like the reference
    ts = sort_like_reference(test)
    want, _ = oracle.rmse_literal(k, ts, Po, Qo, rules)
    got = eng.eval_rmse()
    assert_bit_equal(np.float32(got), np.float32(want), "rmse")
    assert abs(got - oracle.rmse_double(k, ts, Po, Qo)) <= 1e-5 * got      # float64 recomputation, 1e-5 relative
    eng.close()


def mascot_oracle_model(oracle, eng, k, P, Q):
    """Oracle state in the engine's sorted-index space, after checking that the engine's
    m-quantization set-up equals the oracle's restatement of the reference preprocessing."""
    u2s, i2s = eng.index_maps()
    uend, uprec, _ = eng.group_info(0)
    iend, iprec, _ = eng.group_info(1)
    ug = np.searchsorted(uend, np.arange(eng.n_users), side="left").astype(np.uint32)
    ig = np.searchsorted(iend, np.arange(eng.n_items), side="left").astype(np.uint32)
    Ps = np.empty_like(P); Ps[u2s] = P
    Qs = np.empty_like(Q); Qs[i2s] = Q
    return oracle.MascotModel(k, Ps, Qs, ug, ig, uprec, iprec), u2s, i2s


@pytest.mark.parametrize("k", KS)
def test_mascot_training_with_switching_bit_exact(mascot, oracle, k):
    """Seven epochs of the MASCOT variant in deterministic mode: preprocessing, all four precision
    cases (after forced and threshold-driven promotions), the sampled statistics of the check
    epochs, the group errors and the switching decisions - all equal to the oracle."""
    rng = np.random.default_rng(7 + k)
    n_users, n_items, n = 403, 301, 9000
    wu = np.arange(1, n_users + 1) ** -0.9; wi = np.arange(1, n_items + 1) ** -1.1
    R = np.empty(n, mascot.RATING)
    R["u"] = rng.choice(n_users, n, p=wu / wu.sum())
    R["i"] = rng.choice(n_items, n, p=wi / wi.sum())
    R["u"][:n_users] = np.arange(n_users); R["i"][:n_items] = np.arange(n_items)   # everyone rated once
    R["r"] = rng.choice(np.arange(0.5, 5.01, 0.5), n)
    R = R[rng.permutation(n)]
    P = (rng.standard_normal((n_users, k)) * 0.2).astype(np.float32)
    Q = (rng.standard_normal((n_items, k)) * 0.2).astype(np.float32)
    test = R[rng.permutation(n)[:1500]]
    threshold = 0.9
    eng = make_engine(mascot, mascot.V_MASCOT, k, lam=0.015, user_group_num=12, item_group_num=9,
                      sample_ratio=0.3, interval=1, error_threshold=threshold)
    eng.set_ratings(R, test, n_users, n_items)
    eng.set_factors(P, Q)

    # preprocessing parity (degree sort, grouping, maps)
    s2o, o2s, cnt = oracle.degree_sort(R["u"], n_users)
    uend_o, _ = oracle.grouping(cnt, 12)
    s2o_i, o2s_i, cnt_i = oracle.degree_sort(R["i"], n_items)
    iend_o, _ = oracle.grouping(cnt_i, 9)
    model, u2s, i2s = mascot_oracle_model(oracle, eng, k, P, Q)
    assert (u2s == o2s).all() and (i2s == o2s_i).all()
    assert (eng.group_info(0)[0] == uend_o).all() and (eng.group_info(1)[0] == iend_o).all()

    Rs = R.copy(); Rs["u"] = u2s[R["u"]]; Rs["i"] = i2s[R["i"]]
    lrs = oracle.lr_schedule(0.01, 0.1, 50)
    rules = oracle.rules_reference()
    ug, ig = len(uend_o), len(iend_o)
    init_u, init_i = np.ones(ug, np.float32), np.ones(ig, np.float32)
    sample_num = int(np.float32(n) * np.float32(0.3))
    promoted_any = False
    for e in range(8):
        if e == 2:      # force a mix of precisions early so that all four cases run
            for side, g in ((0, 1), (0, ug - 1), (1, 0), (1, ig - 2)):
                eng.promote_group(side, g)
                model.promote("u" if side == 0 else "i", g)
        check = oracle.is_check_epoch(e, 50, 1)
        st = eng.train_epoch(e)
        assert bool(st.error_check) == check
        stats = model.run(Rs, None, float(lrs[e]), 0.015, rules,
                          first_sample_pos=(n - sample_num) if check else None, stats=check, item_stats_by_run=True)
        if check:
            got = eng.sample_stats()
            for a, b, what in zip(got, stats, ("gsum_p", "gsum_q", "nsum_p", "nsum_q")):
                assert_bit_equal(a, b, f"epoch {e} {what}")
            eu = oracle.group_errors(stats[0], stats[2], k, model.uprec, init_u)
            ei = oracle.group_errors(stats[1], stats[3], k, model.iprec, init_i)
            assert_bit_equal(eng.group_info(0)[2], eu, "user group errors")
            assert_bit_equal(eng.group_info(1)[2], ei, "item group errors")
            if e == 5:
                init_u, init_i = eu.copy(), ei.copy()
            else:
                nu_p = ni_p = 0
                for g in range(ug):
                    if eu[g] > threshold and not model.uprec[g]:
                        model.promote("u", g); nu_p += 1
                for g in range(ig):
                    if ei[g] > threshold and not model.iprec[g]:
                        model.promote("i", g); ni_p += 1
                assert (st.promoted_user_groups, st.promoted_item_groups) == (nu_p, ni_p)
                promoted_any |= (nu_p + ni_p) > 0
        assert (eng.group_info(0)[1] == model.uprec).all() and (eng.group_info(1)[1] == model.iprec).all()
        Pg, Qg = eng.get_factors(1)
        Po, Qo = model.factors()
        assert_bit_equal(Pg, Po, f"epoch {e} P")
        assert_bit_equal(Qg, Qo, f"epoch {e} Q")
    assert promoted_any, "the case is meant to exercise threshold-driven switching"
    # evaluation straight from the mixed-precision arenas
    ts = sort_like_reference(test); ts_s = ts.copy(); ts_s["u"] = u2s[ts["u"]]; ts_s["i"] = i2s[ts["i"]]
    want, _ = oracle.rmse_literal(k, ts_s, Po, Qo, rules)
    assert_bit_equal(np.float32(eng.eval_rmse()), np.float32(want), "rmse")
    got_test = eng.test_ratings(1)
    assert (got_test["u"] == ts_s["u"]).all() and (got_test["i"] == ts_s["i"]).all() and (got_test["r"] == ts_s["r"]).all()
    # compact-id view is the permuted sorted view
    P0, Q0 = eng.get_factors(0)
    assert_bit_equal(P0, Po[u2s], "P order 0")
    assert_bit_equal(Q0, Qo[i2s], "Q order 0")
    eng.close()


def assert_within_one_ulp(got, want, half_storage, what):
    """old + (new - old) against new: exact unless new - old is not representable, and then off by at
    most half an ulp of the LARGER of old and new.  Bound used: one ulp (of the storage format) of the
    largest magnitude in the matrix; and all but 3 % of the values must be exactly equal."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    eps = 2.0 ** -10 if half_storage else 2.0 ** -23
    d = np.abs(got - want)
    assert d.max() <= eps * np.abs(want).max(), f"{what}: largest difference {d.max():.3e}"
    assert (d != 0).mean() <= 0.03, f"{what}: {(d != 0).mean():.4f} of the values differ"


@pytest.mark.parametrize("k", KS)
@pytest.mark.parametrize("plain_stores", [1, 0])
@pytest.mark.parametrize("version", ["sgd", "mascot_hh", "mascot_fh", "mascot_hf", "mascot_ff"])
def test_full_grid_on_conflict_free_ratings_bit_exact(mascot, oracle, k, version, plain_stores):
    """Throughput mode (persistent grid, shuffled stream): when no two ratings share a user or an
    item the result does not depend on the schedule, so the Hogwild kernel must equal the oracle -
    bit for bit with plain stores; with the default write-back of user rows (a reduction of the
    change) a user value may differ by one ulp where new - old is not exactly representable."""
    rng = np.random.default_rng(11 + k)
    n = 20011
    R = np.empty(n, mascot.RATING)
    R["u"] = rng.permutation(n); R["i"] = rng.permutation(n)
    R["r"] = rng.choice(np.arange(1, 6), n)
    P = (rng.standard_normal((n, k)) * 0.2).astype(np.float32)
    Q = (rng.standard_normal((n, k)) * 0.2).astype(np.float32)
    vid = mascot.V_SGD if version == "sgd" else mascot.V_MASCOT
    eng = make_engine(mascot, vid, k, deterministic=0, shuffle=1, seed=99, user_group_num=10, item_group_num=10,
                      plain_user_stores=plain_stores)
    eng.set_ratings(R, R[:100], n, n)
    eng.set_factors(P, Q)
    # every entity has degree 1, so each side is a single group: promoting it switches the whole side
    model = None
    if version != "sgd":
        model, u2s, i2s = mascot_oracle_model(oracle, eng, k, P, Q)
        if version in ("mascot_fh", "mascot_ff"):
            eng.promote_group(0, 0); model.promote("u", 0)
        if version in ("mascot_hf", "mascot_ff"):
            eng.promote_group(1, 0); model.promote("i", 0)
    st = eng.train_epoch(0)
    assert st.updates == n
    rules = oracle.rules_reference()
    if version == "sgd":
        Po, Qo = P.copy(), Q.copy()
        oracle.sgd_run(k, R, None, Po, Qo, 0.01, 0.05, rules)
        Pg, Qg = eng.get_factors(0)
    else:
        Rs = R.copy(); Rs["u"] = u2s[R["u"]]; Rs["i"] = i2s[R["i"]]
        model.run(Rs, None, 0.01, 0.05, rules)
        Po, Qo = model.factors()
        Pg, Qg = eng.get_factors(1)
    if plain_stores:
        assert_bit_equal(Pg, Po, "P")
    else:
        assert_within_one_ulp(Pg, Po, version in ("mascot_hh", "mascot_hf"), "P")
    assert_bit_equal(Qg, Qo, "Q")
    eng.close()


def test_seeded_shuffle_is_a_permutation_and_is_followed(mascot, oracle):
    rng = np.random.default_rng(3)
    k, n_users, n_items, n = 64, 90, 70, 3001
    R, P, Q = random_problem(rng, n_users, n_items, n, k)
    eng = make_engine(mascot, mascot.V_SGD, k, shuffle=1, seed=1234)
    eng.set_ratings(R, R[:10], n_users, n_items)
    eng.set_factors(P, Q)
    order = eng.stream_order().astype(np.int64)
    assert [eng.stream_source_index(j) for j in (0, 1, 77, n - 1)] == [order[0], order[1], order[77], order[n - 1]]
    assert sorted(order.tolist()) == list(range(n)) and (order != np.arange(n)).any()
    items = R["i"][order]
    assert (np.diff(items.astype(np.int64)) >= 0).all(), "one window (n < 4096): equal items are neighbours"
    eng.train_epoch(0)
    Po, Qo = P.copy(), Q.copy()
    oracle.sgd_run(k, R, order.astype(np.uint32), Po, Qo, 0.01, 0.05, oracle.rules_reference())
    Pg, Qg = eng.get_factors(0)
    assert_bit_equal(Pg, Po, "P"); assert_bit_equal(Qg, Qo, "Q")
    eng2 = make_engine(mascot, mascot.V_SGD, k, shuffle=1, seed=1235)
    eng2.set_ratings(R, R[:10], n_users, n_items)
    assert any(eng2.stream_source_index(j) != order[j] for j in range(50)), "the seed changes the order"
    eng.close(); eng2.close()


# --------------------------------------------------------------------------------------------
# edge cases and error behaviour
# --------------------------------------------------------------------------------------------
def test_edge_cases(mascot, oracle):
    k = 64
    rng = np.random.default_rng(1)
    R, P, Q = random_problem(rng, 8, 6, 1, k)          # a single rating
    eng = make_engine(mascot, mascot.V_SGD, k)
    with pytest.raises(mascot.MascotError) as e:
        eng.train_epoch(0)
    assert e.value.status == mascot.ERR_STATE
    eng.set_ratings(R, R[:0], 8, 6)                   # empty test set
    with pytest.raises(mascot.MascotError) as e:
        eng.train_epoch(0)                            # factors missing
    assert e.value.status == mascot.ERR_STATE
    eng.set_factors(P, Q)
    eng.train_epoch(0)
    Po, Qo = P.copy(), Q.copy()
    oracle.sgd_run(k, R, None, Po, Qo, 0.01, 0.05, oracle.rules_reference())
    Pg, Qg = eng.get_factors(0)
    assert_bit_equal(Pg, Po); assert_bit_equal(Qg, Qo)
    with pytest.raises(mascot.MascotError) as e:
        eng.eval_rmse()
    assert e.value.status == mascot.ERR_STATE
    # empty training set: an epoch is a no-op
    eng.set_ratings(R[:0], R, 8, 6)
    eng.set_factors(P, Q)
    assert eng.train_epoch(0).updates == 0
    Pg, Qg = eng.get_factors(0)
    assert_bit_equal(Pg, P); assert_bit_equal(Qg, Q)
    # id out of range
    bad = R.copy(); bad["u"] = 8
    with pytest.raises(mascot.MascotError) as e:
        eng.set_ratings(bad, R, 8, 6)
    assert e.value.status == mascot.ERR_BAD_ARG
    eng.close()
    with pytest.raises(mascot.MascotError) as e:
        mascot.Engine(mascot.default_config(version=mascot.V_SGD, device=77))
    assert e.value.status == mascot.ERR_NO_DEVICE


def test_lr_zero_keeps_fp32_factors_and_init_is_seeded(mascot):
    k, n_users, n_items, n = 128, 3000, 1000, 200000
    rng = np.random.default_rng(2)
    R, _, _ = random_problem(rng, n_users, n_items, n, k)
    eng = make_engine(mascot, mascot.V_SGD, k, deterministic=0, shuffle=1, learning_rate=0.0, seed=5)
    eng.set_ratings(R, R[:1000], n_users, n_items)
    eng.init_factors()
    P0, Q0 = eng.get_factors(0)
    assert abs(P0.std() - 0.01) < 5e-4 and abs(P0.mean()) < 1e-4 and abs(Q0.std() - 0.01) < 5e-4
    eng.train_epoch(0)
    P1, Q1 = eng.get_factors(0)
    assert_bit_equal(P0, P1); assert_bit_equal(Q0, Q1)      # p + 0*g == p exactly
    eng.init_factors()
    P2, _ = eng.get_factors(0)
    assert_bit_equal(P0, P2, "same seed, same factors")
    eng.close()


# --------------------------------------------------------------------------------------------
# MuPPET (-v 3)
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", [f"muppet_k{k}_b{b}" for k in KS for b in (8, 12, 14, 16, 32)])
def test_golden_muppet(mascot, oracle, golden, name):
    """The reference kernel's factors and both sampled statistics, at every pass width."""
    I, G = golden
    c = golden_case(I, G, name, oracle)
    seq = c["seq"]
    n = len(seq)
    train = mascot.as_ratings(np.ascontiguousarray(c["R"][seq]))
    ratio = (n - c["fs"] + 0.01) / n                       # the engine samples the last int(n * ratio) ratings
    assert int(np.float32(n) * np.float32(ratio)) == n - c["fs"]
    eng = make_engine(mascot, mascot.V_MUPPET, c["k"], learning_rate=c["lr"], lam=c["lam"], sample_ratio=ratio,
                      muppet_width=c["extra0"])
    eng.set_ratings(train, train[:1], c["nu"], c["ni"])
    eng.set_factors(c["P"], c["Q"])
    st = eng.train_epoch(0)
    assert st.pass_bits == c["extra0"]
    P, Q = eng.get_factors(0)
    gp, _gq, np_, _nq = eng.sample_stats()
    eng.close()
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")
    assert_bit_equal(gp[:c["k"]], G[name + ".sum_updated_val"], "sum_updated_val")
    assert_bit_equal(np_[:1], G[name + ".sum_norms"], "sum_norms")


def muppet_policy_step(state, e, k, sums, norm):
    """mf_methods.cu:602, 660-695 restated: returns the index into (8, 12, 14, 16, 32) for the next epoch."""
    state["norms"].append(np.float32(norm)); state["sums"].append(np.asarray(sums, np.float32).copy())
    thr = np.float32(1.0) + np.float32(1.5) * np.exp(np.float32(-1 * np.float32(0.3) * e), dtype=np.float32)
    if e - state["switched"] < 3:
        return
    norms = np.float32(0)
    acc = np.zeros(k, np.float32)
    for w in range(e - 2, e + 1):
        norms = np.float32(norms + state["norms"][w]); acc = (acc + state["sums"][w]).astype(np.float32)
    sq = np.float32(0)
    for d in range(k):
        sq = np.float32(sq + np.float32(acc[d]) * np.float32(acc[d]))
    with np.errstate(all="ignore"):
        div = np.float32(norms) / np.float32(sq)
        state["max"] = div if state["max"] < div else state["max"]
        ratio = np.float32(state["max"]) / div
    if ratio > thr:
        state["idx"] = min(state["idx"] + 1, 4); state["switched"] = e; state["max"] = np.float32(-1)


@pytest.mark.parametrize("k,start_width,scale,switch_expected", [(64, 0, 0.1, True), (128, 14, 0.2, False)])
def test_muppet_epochs_with_width_policy_bit_exact(mascot, oracle, k, start_width, scale, switch_expected):
    """Twelve deterministic epochs of -v 3: every epoch's factors and statistics come from the oracle's
    restatement at the width the host policy chose, and the engine must choose the same widths.  The
    k=64 problem crosses the 8 -> 12 bit switch at epoch 7; the k=128 run starts at 14 bits."""
    rng = np.random.default_rng(300 + k)
    n_users, n_items, n = 97, 83, 3001
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=scale)
    eng = make_engine(mascot, mascot.V_MUPPET, k, sample_ratio=0.25, learning_rate=0.03, muppet_width=start_width)
    eng.set_ratings(R, R[:300], n_users, n_items)
    eng.set_factors(P, Q)
    lrs = oracle.lr_schedule(0.03, 0.1, 50)
    rules = oracle.rules_reference()
    Po, Qo = P.copy(), Q.copy()
    widths = (8, 12, 14, 16, 32)
    state = dict(idx=widths.index(start_width) if start_width else 0, switched=-1, max=np.float32(-1), norms=[], sums=[])
    fsp = n - int(np.float32(n) * np.float32(0.25))
    seen = []
    for e in range(12):
        bits = widths[state["idx"]]
        st = eng.train_epoch(e)
        assert st.pass_bits == bits, f"epoch {e}: engine ran {st.pass_bits} bits, policy says {bits}"
        seen.append(bits)
        suv, sn = oracle.muppet_run(k, R, None, Po, Qo, float(lrs[e]), 0.05, bits, bits, rules, first_sample_pos=fsp)
        assert np.isfinite(Po).all() and np.isfinite(Qo).all()
        gp, _gq, np_, _nq = eng.sample_stats()
        assert_bit_equal(gp[:k], suv, f"sum_updated_val epoch {e}")
        assert_bit_equal(np_[:1], np.float32(sn), f"sum_norms epoch {e}")
        muppet_policy_step(state, e, k, suv, sn)
    Pg, Qg = eng.get_factors(0)
    eng.close()
    assert_bit_equal(Pg, Po, "P")
    assert_bit_equal(Qg, Qo, "Q")
    if switch_expected:
        assert len(set(seen)) > 1, "the run should cross at least one width switch"


# --------------------------------------------------------------------------------------------
# AFP (-v 2)
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", [f"afp_k{k}_e{e}" for k in KS for e in (0, 1)])
def test_golden_afp(mascot, oracle, golden, name):
    """The reference kernel's factors; the golden case's epoch index is reproduced by a schedule
    without decay, so that epoch 1 runs at the case's learning rate as well."""
    I, G = golden
    c = golden_case(I, G, name, oracle)
    seq = c["seq"]
    train = mascot.as_ratings(np.ascontiguousarray(c["R"][seq]))
    eng = make_engine(mascot, mascot.V_AFP, c["k"], learning_rate=c["lr"], lam=c["lam"], decay=0.0)
    eng.set_ratings(train, train[:1], c["nu"], c["ni"])
    eng.set_factors(c["P"], c["Q"])
    st = eng.train_epoch(c["extra0"])
    assert st.updates == len(seq) and np.float32(st.lr) == np.float32(c["lr"])
    P, Q = eng.get_factors(0)
    eng.close()
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


@pytest.mark.parametrize("k", KS)
def test_afp_epochs_bit_exact(mascot, oracle, k):
    """Four deterministic epochs of -v 2 on a ragged problem: the worker's format state (8/16 bits per
    side, re-estimation intervals) must follow the oracle's restatement rating by rating."""
    rng = np.random.default_rng(400 + k)
    n_users, n_items, n = 131, 89, 4003
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=0.2)
    eng = make_engine(mascot, mascot.V_AFP, k)
    eng.set_ratings(R, R[:300], n_users, n_items)
    eng.set_factors(P, Q)
    lrs = oracle.lr_schedule(0.01, 0.1, 50)
    rules = oracle.rules_reference()
    Po, Qo = P.copy(), Q.copy()
    threshold = int(np.float32(n) / np.float32(10.0))
    for e in range(4):
        eng.train_epoch(e)
        oracle.afp_run(k, R, None, Po, Qo, float(lrs[e]), 0.05, e, threshold, rules)
    Pg, Qg = eng.get_factors(0)
    eng.close()
    assert np.isfinite(Po).all()
    assert_bit_equal(Pg, Po, "P")
    assert_bit_equal(Qg, Qo, "Q")


# --------------------------------------------------------------------------------------------
# replacing the training stream, stream handle
# --------------------------------------------------------------------------------------------
def test_reload_train_replaces_the_stream(mascot, oracle):
    """mascot_reload_train: the next epoch runs over the new ratings (same and different length), with
    the factors it already has."""
    rng = np.random.default_rng(77)
    k, n_users, n_items = 64, 60, 50
    R1, P, Q = random_problem(rng, n_users, n_items, 1500, k)
    R2, _, _ = random_problem(rng, n_users, n_items, 1500, k)
    R3, _, _ = random_problem(rng, n_users, n_items, 777, k)
    eng = make_engine(mascot, mascot.V_SGD, k)
    eng.set_ratings(R1, R1[:100], n_users, n_items)
    eng.set_factors(P, Q)
    lrs = oracle.lr_schedule(0.01, 0.1, 50)
    rules = oracle.rules_reference()
    Po, Qo = P.copy(), Q.copy()
    for e, R in enumerate((R1, R2, R3)):
        if e:
            eng.reload_train(R)
        st = eng.train_epoch(e)
        assert st.updates == R.size
        oracle.sgd_run(k, R, None, Po, Qo, float(lrs[e]), 0.05, rules)
    Pg, Qg = eng.get_factors(0)
    eng.close()
    assert_bit_equal(Pg, Po, "P")
    assert_bit_equal(Qg, Qo, "Q")


def test_stream_handle_orders_caller_work(mascot):
    """mascot_get_stream: a torch copy queued on the engine's stream sees the factors of the epoch
    queued before it without any host-side wait in between."""
    import torch
    rng = np.random.default_rng(5)
    k, n_users, n_items = 64, 40, 30
    R, P, Q = random_problem(rng, n_users, n_items, 900, k)
    eng = make_engine(mascot, mascot.V_SGD, k)
    eng.set_ratings(R, R[:50], n_users, n_items)
    eng.set_factors(P, Q)
    ext = torch.cuda.ExternalStream(eng.stream_handle(), device=torch.device("cuda", 0))
    (p16, b16), (p32, b32) = eng.item_rows(0, n_items)
    assert p16 == 0 and b32 == n_items * k * 4, "the fp32 trainer keeps only the fp32 arena"

    class Raw:
        __cuda_array_interface__ = {"shape": (b32,), "typestr": "|u1", "data": (p32, False), "version": 2}
    view = torch.as_tensor(Raw(), device="cuda:0")
    eng.train_segment(0, 0, wait=False)
    with torch.cuda.stream(ext):
        snap = view.clone()
    ext.synchronize()
    _, Qg = eng.get_factors(0)
    eng.close()
    got = np.sort(snap.cpu().numpy().view(np.float32))
    assert (got == np.sort(Qg.reshape(-1))).all(), "the copy ran after the kernel (same values, row-internal order is the library's)"


def test_streamed_epoch_equals_resident_epoch(mascot, oracle):
    """mascot_train_epoch_streamed on host ratings == mascot_train_epoch on the resident stream, for a
    MASCOT run through its first check epochs (factors, statistics and precisions bit for bit)."""
    rng = np.random.default_rng(91)
    k, n_users, n_items, n = 128, 150, 120, 6001
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=0.2)
    engines = []
    for _ in range(2):
        eng = make_engine(mascot, mascot.V_MASCOT, k, user_group_num=5, item_group_num=4, sample_ratio=0.3, interval=1,
                          error_threshold=0.5)
        eng.set_ratings(R, R[:200], n_users, n_items)
        eng.set_factors(P, Q)
        engines.append(eng)
    a, b = engines
    for e in range(8):
        sa = a.train_epoch(e)
        sb = b.train_epoch_streamed(e, R)
        assert (sa.error_check, sa.promoted_user_groups, sa.promoted_item_groups) == (sb.error_check, sb.promoted_user_groups, sb.promoted_item_groups)
        for x, y in zip(a.sample_stats(), b.sample_stats()):
            assert_bit_equal(x, y, f"statistics epoch {e}")
    for x, y in zip(a.get_factors(1), b.get_factors(1)):
        assert_bit_equal(x, y, "factors")
    assert a.group_info(0)[1].tolist() == b.group_info(0)[1].tolist()
    a.close(); b.close()


def test_streamed_epoch_over_two_pieces_bit_exact(mascot, oracle):
    """A rating array longer than one upload piece (8Mi ratings): the pieces are trained in order, each
    exactly once, and the deterministic result equals the sequential oracle."""
    rng = np.random.default_rng(92)
    k, n_users, n_items = 64, 3000, 2000
    n = (8 << 20) + 1234
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=0.1)
    eng = make_engine(mascot, mascot.V_SGD, k)
    eng.set_ratings(R[:1000], R[:100], n_users, n_items)
    eng.set_factors(P, Q)
    st = eng.train_epoch_streamed(0, R)
    assert st.updates == n
    Pg, Qg = eng.get_factors(0)
    eng.close()
    Po, Qo = P.copy(), Q.copy()
    oracle.sgd_run(k, R, None, Po, Qo, 0.01, 0.05, oracle.rules_reference())
    assert_bit_equal(Pg, Po, "P")
    assert_bit_equal(Qg, Qo, "Q")


# --------------------------------------------------------------------------------------------
# whole-model switching trainer (-v 8) and the naive variant (-v 6)
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["switching_k128_half", "switching_k128_half_big"])
def test_golden_switching_only_half(mascot, oracle, golden, name):
    """The reference kernel's binary16 phase: factors and both sampled statistics.  Epoch index 5 is the
    first check epoch; without decay it runs at the case's learning rate."""
    I, G = golden
    c = golden_case(I, G, name, oracle)
    seq = c["seq"]
    n = len(seq)
    train = mascot.as_ratings(np.ascontiguousarray(c["R"][seq]))
    ratio = (n - c["fs"] + 0.01) / n
    assert int(np.float32(n) * np.float32(ratio)) == n - c["fs"]
    eng = make_engine(mascot, mascot.V_SWITCH_ONLY, c["k"], learning_rate=c["lr"], lam=c["lam"], decay=0.0, sample_ratio=ratio,
                      interval=1, error_threshold=1e30)
    eng.set_ratings(train, train[:1], c["nu"], c["ni"])
    eng.set_factors(c["P"], c["Q"])
    st = eng.train_epoch(5)
    assert st.error_check == 1 and np.float32(st.lr) == np.float32(c["lr"])
    P, Q = eng.get_factors(0)
    gp, _gq, np_, _nq = eng.sample_stats()
    eng.close()
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")
    assert_bit_equal(gp[:c["k"]], G[name + ".sum_updated_val"], "sum_updated_val")
    assert_bit_equal(np_[:1], G[name + ".sum_norms"], "sum_norms")


def test_golden_switching_only_float_phase_is_the_fp32_trainer(mascot, oracle, golden):
    I, G = golden
    name = "switching_k128_float"
    c = golden_case(I, G, name, oracle)
    P, Q = replay_through_engine(mascot, mascot.V_SGD, c)
    assert_bit_equal(P, G[name + ".P_out"], "P")
    assert_bit_equal(Q, G[name + ".Q_out"], "Q")


def test_switching_only_run_with_its_switch_bit_exact(mascot, oracle):
    """Ten deterministic epochs of -v 8 with a threshold that forces the switch: binary16 epochs, the
    error test of mf_methods.cu:1515-1545 on the check epochs, then fp32 epochs - all against the oracle."""
    rng = np.random.default_rng(500)
    k, n_users, n_items, n = 128, 90, 70, 2501
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=0.2)
    threshold = 0.4          # the relative error is 0.51 at epoch 6 on this problem: the switch happens there
    eng = make_engine(mascot, mascot.V_SWITCH_ONLY, k, sample_ratio=0.2, interval=1, error_threshold=threshold, epoch=10)
    eng.set_ratings(R, R[:200], n_users, n_items)
    eng.set_factors(P, Q)
    lrs = oracle.lr_schedule(0.01, 0.1, 10)
    rules = oracle.rules_reference()
    P16, Q16 = oracle.f2h(P), oracle.f2h(Q)
    P32 = Q32 = None
    fsp = n - int(np.float32(n) * np.float32(0.2))
    initial, switched_at = np.float32(1), None
    for e in range(10):
        st = eng.train_epoch(e)
        if P32 is None:
            check = oracle.is_check_epoch(e, 10, 1)
            assert st.error_check == int(check)
            suv, sn = oracle.switching_run(k, R, None, P16, Q16, 0, float(lrs[e]), 0.05, rules, first_sample_pos=fsp if check else None)
            if check:
                sq = np.float32(0)
                for d in range(k):
                    sq = np.float32(sq + np.float32(suv[d]) * np.float32(suv[d]))
                err = np.float32(np.float32(sq / np.float32(sn)) / initial)
                if e == 5:
                    initial = err
                if e > 5 and err > np.float32(threshold):
                    P32, Q32 = oracle.h2f(P16), oracle.h2f(Q16)
                    switched_at = e
                    assert st.promoted_user_groups == 1 and st.promoted_item_groups == 1
                else:
                    assert st.promoted_user_groups == 0
        else:
            assert st.error_check == 0
            oracle.switching_run(k, R, None, P32, Q32, 1, float(lrs[e]), 0.05, rules)
    assert switched_at is not None and switched_at < 9, "the run should cross the switch"
    Pg, Qg = eng.get_factors(0)
    eng.close()
    assert_bit_equal(Pg, P32, "P")
    assert_bit_equal(Qg, Q32, "Q")


@pytest.mark.parametrize("k", KS)
def test_naive_variant_runs_as_mascot(mascot, k):
    """-v 6 is -v 1 with another group lookup in the reference: same engine path, same result."""
    rng = np.random.default_rng(600 + k)
    n_users, n_items, n = 80, 60, 2000
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=0.2)
    out = []
    for v in (mascot.V_MASCOT, mascot.V_NAIVE):
        eng = make_engine(mascot, v, k, user_group_num=4, item_group_num=3, sample_ratio=0.3, interval=1, error_threshold=0.5)
        eng.set_ratings(R, R[:100], n_users, n_items)
        eng.set_factors(P, Q)
        for e in range(7):
            eng.train_epoch(e)
        out.append(eng.get_factors(0))
        eng.close()
    assert_bit_equal(out[0][0], out[1][0], "P")
    assert_bit_equal(out[0][1], out[1][1], "Q")
