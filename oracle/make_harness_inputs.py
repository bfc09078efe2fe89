"""Generate the seeded input bundle for the reference-kernel harness (oracle/ref_harness.cu).

TEST INFRASTRUCTURE ONLY.  Run:  python oracle/make_harness_inputs.py  -> tests/golden/harness_in.bin

Every case is a tiny problem that one warp of a reference training kernel walks through
sequentially; the harness also records the chunk start positions the kernel drew, so the CPU
oracle can replay exactly the same update sequence and be compared bit for bit.

Case kinds: 0 fp32 SGD, 1 MASCOT (mixed fp16/fp32 groups + sampled statistics), 2 MPT,
3 fp16-storage SGD, 4 MuPPET, 5 AFP, 6 test-RMSE, 7 whole-model switching.

A second bundle, tests/golden/setup_in.bin, holds the cases of kind 8: small rating sets (many tied
degrees, unrated entities, a single degree class) on which the harness runs the reference's
m-quantization set-up functions.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from bundle import write_bundle  # noqa: E402

KIND = dict(sgd=0, mascot=1, mpt=2, memquant=3, muppet=4, afp=5, rmse=6, switching=7)


def half_round(a):
    return a.astype(np.float16).astype(np.float32)


def make_ratings(rng, n_users, n_items, nnz, grid):
    u = rng.integers(0, n_users, nnz).astype(np.uint32)
    i = rng.integers(0, n_items, nnz).astype(np.uint32)
    r = rng.choice(grid, nnz).astype(np.float32)
    out = np.empty((nnz, 3), np.uint32)
    out[:, 0] = r.view(np.uint32)
    out[:, 1] = u
    out[:, 2] = i
    return out


def end_idx_from_sizes(sizes):
    return (np.cumsum(sizes) - 1).astype(np.uint32)


def training_case(rng, kind, k, n_users, n_items, nnz, update_count, vector_size, first_sample,
                  seed, lr, lam, scale=0.1, extra0=0, extra1=0, grid=None, half_rows=False):
    grid = np.arange(0.5, 5.01, 0.5) if grid is None else grid
    P = (rng.standard_normal((n_users, k)) * scale).astype(np.float32)
    Q = (rng.standard_normal((n_items, k)) * scale).astype(np.float32)
    if half_rows:
        P, Q = half_round(P), half_round(Q)
    return {
        "meta": np.array([KIND[kind], k, n_users, n_items, nnz, update_count, vector_size,
                          first_sample, seed, extra0, extra1], np.int32),
        "hyper": np.array([lr, lam], np.float32),
        "R": make_ratings(rng, n_users, n_items, nnz, grid),
        "P": P,
        "Q": Q,
    }


def mascot_case(rng, k, usizes, isizes, uprec, iprec, nnz, update_count, vector_size,
                first_sample, seed, lr, lam, scale=0.1):
    n_users, n_items = int(sum(usizes)), int(sum(isizes))
    c = training_case(rng, "mascot", k, n_users, n_items, nnz, update_count, vector_size,
                      first_sample, seed, lr, lam, scale)
    uend, iend = end_idx_from_sizes(usizes), end_idx_from_sizes(isizes)
    # rows of fp16 groups start out exactly representable in binary16
    ug = np.searchsorted(uend, np.arange(n_users), side="left")
    ig = np.searchsorted(iend, np.arange(n_items), side="left")
    uprec, iprec = np.asarray(uprec, np.uint8), np.asarray(iprec, np.uint8)
    c["P"][uprec[ug] == 0] = half_round(c["P"][uprec[ug] == 0])
    c["Q"][iprec[ig] == 0] = half_round(c["Q"][iprec[ig] == 0])
    c.update(uend=uend, iend=iend, uprec=uprec, iprec=iprec)
    return c


def rmse_case(rng, k, n_users, n_items, n_test):
    c = training_case(rng, "rmse", k, n_users, n_items, n_test, 0, 0, 0, 0, 0.0, 0.0, scale=0.15)
    return c


def tight_ratings(rng, c, matching):
    """Replace the ratings of a case by the exact prediction plus a tiny perturbation."""
    k = int(c["meta"][1])
    n = int(c["meta"][4])
    if matching:
        u = rng.permutation(int(c["meta"][2]))[:n].astype(np.uint32)
        i = rng.permutation(int(c["meta"][3]))[:n].astype(np.uint32)
    else:
        u, i = c["R"][:, 1].copy(), c["R"][:, 2].copy()
    pred = np.einsum("nk,nk->n", c["P"][u].astype(np.float64), c["Q"][i].astype(np.float64))
    r = (pred * (1.0 + rng.standard_normal(n) * 1e-5)).astype(np.float32)
    c["R"][:, 0] = r.view(np.uint32)
    c["R"][:, 1] = u
    c["R"][:, 2] = i


def setup_case(rng, k, n_users, n_items, nnz, n_test, ug, ig, zipf=None, unrated=(0, 0), flat=False):
    """Ratings for the set-up pipeline: users/items drawn uniformly or by a power law; the last
    `unrated` users/items never occur; `flat` gives every user the same degree."""
    ru, ri = n_users - unrated[0], n_items - unrated[1]
    if flat:
        u = np.repeat(np.arange(ru, dtype=np.uint32), nnz // ru)
        nnz = u.size
        i = rng.integers(0, ri, nnz).astype(np.uint32)
    else:
        def draw(n, count):
            if zipf is None:
                return rng.integers(0, n, count)
            w = np.arange(1, n + 1, dtype=np.float64) ** -zipf
            return rng.permutation(n)[rng.choice(n, size=count, p=w / w.sum())]
        u = np.concatenate([np.arange(ru), draw(ru, nnz - ru)]).astype(np.uint32)
        i = np.concatenate([np.arange(ri), draw(ri, nnz - ri)])[rng.permutation(nnz)].astype(np.uint32)
    R = np.empty((nnz, 3), np.uint32)
    R[:, 0] = rng.choice(np.arange(0.5, 5.01, 0.5), nnz).astype(np.float32).view(np.uint32)
    R[:, 1], R[:, 2] = u, i
    T = np.empty((n_test, 3), np.uint32)
    T[:, 0] = rng.choice(np.arange(0.5, 5.01, 0.5), n_test).astype(np.float32).view(np.uint32)
    T[:, 1], T[:, 2] = rng.integers(0, ru, n_test), rng.integers(0, ri, n_test)
    return {
        "meta": np.array([8, k, n_users, n_items, nnz, n_test, ug, ig], np.int32),
        "R": R, "T": T,
        "P": (rng.standard_normal((n_users, k)) * 0.1).astype(np.float32),
        "Q": (rng.standard_normal((n_items, k)) * 0.1).astype(np.float32),
    }


def write_cases(cases, filename):
    arrays = {"cases": np.frombuffer("\n".join(cases).encode(), np.uint8)}
    for name, c in cases.items():
        for key, arr in c.items():
            arrays[f"{name}.{key}"] = arr
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "tests", "golden", filename)
    write_bundle(out, arrays)
    print("wrote", os.path.normpath(out), len(cases), "cases")


def setup_main():
    rng = np.random.default_rng(20211208)
    cases = {
        "setup_tiny_k128": setup_case(rng, 128, 37, 23, 150, 40, 5, 4),
        "setup_zipf_k64": setup_case(rng, 64, 2000, 500, 30000, 300, 100, 100, zipf=1.0),
        "setup_unrated_k128": setup_case(rng, 128, 60, 40, 300, 50, 6, 6, unrated=(10, 5)),
        "setup_flat_k64": setup_case(rng, 64, 16, 8, 64, 20, 4, 3, flat=True),
        "setup_manygroups_k128": setup_case(rng, 128, 300, 200, 4000, 100, 300, 150, zipf=0.8),
    }
    write_cases(cases, "setup_in.bin")


def main():
    rng = np.random.default_rng(20211207)
    cases = {}
    for k in (128, 64):
        t = f"k{k}"
        cases[f"sgd_{t}"] = training_case(rng, "sgd", k, 23, 17, 40, 3, 16, 0, 11, 0.01, 0.05)
        cases[f"sgd_{t}_big"] = training_case(rng, "sgd", k, 50, 40, 300, 4, 128, 0, 12, 0.05, 0.015, scale=0.3)
        cases[f"mascot_{t}_mixed"] = mascot_case(
            rng, k, [5, 4, 7, 3, 5], [6, 3, 4, 7], [0, 1, 0, 1, 0], [0, 0, 1, 1],
            nnz=60, update_count=3, vector_size=32, first_sample=40, seed=21, lr=0.01, lam=0.015)
        cases[f"mascot_{t}_half"] = mascot_case(
            rng, k, [8, 8, 8], [10, 10], [0, 0, 0], [0, 0],
            nnz=50, update_count=2, vector_size=64, first_sample=0, seed=22, lr=0.02, lam=0.05, scale=0.3)
        cases[f"mascot_{t}_float"] = mascot_case(
            rng, k, [6, 6], [5, 5, 5], [1, 1], [1, 1, 1],
            nnz=30, update_count=2, vector_size=24, first_sample=0, seed=23, lr=0.01, lam=0.05)
        cases[f"mpt_{t}"] = training_case(rng, "mpt", k, 19, 21, 45, 3, 20, 0, 31, 0.01, 0.05, half_rows=True)
        cases[f"memquant_{t}"] = training_case(rng, "memquant", k, 19, 21, 45, 3, 20, 0, 41, 0.01, 0.05, half_rows=True)
        for bits in (8, 12, 14, 16, 32):
            cases[f"muppet_{t}_b{bits}"] = training_case(
                rng, "muppet", k, 15, 13, 36, 2, 24, 10, 50 + bits, 0.01, 0.05, extra0=bits)
        for epoch in (0, 1):
            cases[f"afp_{t}_e{epoch}"] = training_case(
                rng, "afp", k, 15, 13, 36, 2, 40, 0, 70 + epoch, 0.01, 0.05, extra0=epoch)
        cases[f"rmse_{t}"] = rmse_case(rng, k, 64, 48, 1300)

    # Second batch: cases built to expose last-bit differences that the first batch hides.
    for k in (128, 64):
        t = f"k{k}"
        # many sampled ratings whose gradients are full fp32 values (mixed precision)
        cases[f"mascot_{t}_mixed_big"] = mascot_case(
            rng, k, [10, 10, 10, 10], [10, 10, 10, 10], [0, 1, 0, 1], [1, 0, 1, 0],
            nnz=400, update_count=4, vector_size=128, first_sample=0, seed=24, lr=0.01, lam=0.015, scale=0.3)
        # ratings that almost equal the current prediction: the residual then carries the low
        # bits of the dot product, and every rating touches rows of its own
        for kind, half_rows in (("memquant", True), ("sgd", False)):
            c = training_case(rng, kind, k, 200, 200, 200, 2, 100, 0, 42, 0.05, 0.05, scale=0.3, half_rows=half_rows)
            tight_ratings(rng, c, matching=True)
            cases[f"{kind}_{t}_tight"] = c
        c = rmse_case(rng, k, 64, 48, 1300)
        tight_ratings(rng, c, matching=False)
        cases[f"rmse_{t}_tight"] = c

    # Third batch (appended, so that the random stream of the cases above stays what it was): the
    # whole-model switching trainer (-v 8, k=128 only in the reference), before and after its switch.
    cases["switching_k128_half"] = training_case(rng, "switching", 128, 15, 13, 36, 2, 24, 10, 81, 0.01, 0.05,
                                                 extra0=0, half_rows=True)
    cases["switching_k128_half_big"] = training_case(rng, "switching", 128, 40, 30, 300, 3, 100, 120, 82, 0.02, 0.015,
                                                     scale=0.3, extra0=0, half_rows=True)
    cases["switching_k128_float"] = training_case(rng, "switching", 128, 15, 13, 36, 2, 24, 10, 83, 0.01, 0.05, extra0=1)

    write_cases(cases, "harness_in.bin")


if __name__ == "__main__":
    main()
    setup_main()
