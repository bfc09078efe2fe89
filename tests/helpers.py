"""Shared helpers of the parity tests."""
import numpy as np


def bits(a):
    return np.ascontiguousarray(a, np.float32).reshape(-1).view(np.uint32)


def assert_bit_equal(a, b, what=""):
    a, b = bits(a), bits(b)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    bad = np.flatnonzero(a != b)
    assert bad.size == 0, f"{what}: {bad.size} of {a.size} values differ, first at {bad[:5]}"


def golden_case(I, G, name, O):
    meta, hy = I[name + ".meta"], I[name + ".hyper"]
    c = dict(kind=int(meta[0]), k=int(meta[1]), nu=int(meta[2]), ni=int(meta[3]), nnz=int(meta[4]), uc=int(meta[5]),
             vec=int(meta[6]), fs=int(meta[7]), extra0=int(meta[9]), lr=float(hy[0]), lam=float(hy[1]))
    c["R"] = I[name + ".R"].reshape(-1, 3)
    c["P"] = I[name + ".P"].reshape(c["nu"], -1)
    c["Q"] = I[name + ".Q"].reshape(c["ni"], -1)
    if name + ".start_ids" in G:
        c["seq"] = O.chunk_sequence(G[name + ".start_ids"], c["vec"], c["nnz"])
    return c


def golden_mascot_model(I, name, c, O):
    uend, iend = I[name + ".uend"], I[name + ".iend"]
    ug = np.searchsorted(uend, np.arange(c["nu"]), side="left").astype(np.uint32)
    ig = np.searchsorted(iend, np.arange(c["ni"]), side="left").astype(np.uint32)
    return O.MascotModel(c["k"], c["P"], c["Q"], ug, ig, I[name + ".uprec"], I[name + ".iprec"])


def random_problem(rng, n_users, n_items, n, k, scale=0.1, grid=None):
    grid = np.arange(0.5, 5.01, 0.5) if grid is None else grid
    R = np.empty(n, np.dtype([("r", np.float32), ("u", np.uint32), ("i", np.uint32)]))
    R["u"] = rng.integers(0, n_users, n)
    R["i"] = rng.integers(0, n_items, n)
    R["r"] = rng.choice(grid, n)
    P = (rng.standard_normal((n_users, k)) * scale).astype(np.float32)
    Q = (rng.standard_normal((n_items, k)) * scale).astype(np.float32)
    return R, P, Q


def sort_like_reference(test):
    """Order of test_set_preprocess (preprocess_utils.h:38-52): by user, then item; equal pairs keep
    the caller's order (the engine uses a stable sort)."""
    return test[np.lexsort((test["i"], test["u"]))]
