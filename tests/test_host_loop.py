"""CPU test of the fast host-core baseline (oracle/host_loop.cpp) that bench.py times: it is checked
against the bit-exact oracle by RMSE, not bit for bit (hardware binary16 conversions, another summation
order, fused multiply-adds that round twice).  Tolerance: 0.5 % relative on the training-fit RMSE after
the same number of sequential epochs, the criterion the engine itself is held to against the reference."""
import numpy as np
import pytest

from helpers import random_problem


def _rmse(P, Q, R):
    pred = np.einsum("nk,nk->n", P[R["u"]].astype(np.float64), Q[R["i"]].astype(np.float64))
    return float(np.sqrt(np.mean((R["r"] - pred) ** 2)))


@pytest.mark.parametrize("k,half", [(128, True), (64, True), (128, False), (64, False)])
def test_host_loop_tracks_the_oracle(oracle, k, half):
    try:
        oracle.host_loop()
    except OSError as e:
        pytest.skip(str(e))
    rng = np.random.default_rng(7 + k)
    n_users, n_items, n = 300, 200, 12000
    R, P, Q = random_problem(rng, n_users, n_items, n, k, scale=0.1)
    fast = oracle.HostLoopModel(k, P, Q, half)
    rules = oracle.rules_reference()
    if half:
        ref = oracle.MascotModel(k, P, Q, np.zeros(n_users, np.uint32), np.zeros(n_items, np.uint32), np.zeros(1, np.uint8), np.zeros(1, np.uint8))
    else:
        Pr, Qr = P.copy(), Q.copy()
    lrs = oracle.lr_schedule(0.02, 0.1, 6)
    for e in range(6):
        fast.epoch(R, float(lrs[e]), 0.05, 1)                     # one thread: the same sequential order as the oracle
        if half:
            ref.run(R, None, float(lrs[e]), 0.05, rules)
        else:
            oracle.sgd_run(k, R, None, Pr, Qr, float(lrs[e]), 0.05, rules)
    Pf, Qf = fast.factors()
    Po, Qo = ref.factors() if half else (Pr, Qr)
    a, b = _rmse(Pf, Qf, R), _rmse(Po, Qo, R)
    assert b < 0.97 * _rmse(P, Q, R), "the problem trains"
    assert abs(a - b) <= 0.005 * b, (a, b)
    # the factors themselves stay close: a few binary16 ulps after six epochs
    assert np.abs(Pf - Po).max() <= 0.02 * np.abs(Po).max()


def test_host_loop_threads_do_not_lose_ratings(oracle):
    """Several threads race on the rows like the GPU workers; the fit must still improve every epoch."""
    try:
        oracle.host_loop()
    except OSError as e:
        pytest.skip(str(e))
    rng = np.random.default_rng(3)
    R, P, Q = random_problem(rng, 2000, 1500, 200000, 128, scale=0.1)
    m = oracle.HostLoopModel(128, P, Q, True)
    before = _rmse(P, Q, R)
    for e in range(3):
        m.epoch(R, 0.02, 0.05, 4)
    Pf, Qf = m.factors()
    assert _rmse(Pf, Qf, R) < 0.95 * before
