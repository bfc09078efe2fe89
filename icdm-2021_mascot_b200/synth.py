"""Seeded synthetic rating matrices with the shapes and value distributions of the benchmark
configurations (stand-ins for ML10M / ML25M / Netflix / Yahoo!Music, which cannot be shipped).

Users and items get power-law (Zipf) or log-normal popularity weights; (user, item) pairs are
drawn from the product of the two marginals without duplicates; ratings come from rank-16
ground-truth factors plus Gaussian noise, mapped onto the rating grid of the configuration.

Two back ends produce the same kind of data: numpy (CPU, any size that fits in host memory) and
torch on a CUDA device (used for the 100M+ configurations, where the numpy path takes minutes).
"""
import numpy as np

RATING = np.dtype([("r", np.float32), ("u", np.uint32), ("i", np.uint32)])

# name -> shape / size / distributions, following the benchmark configuration list
CONFIGS = {
    "c1": dict(users=10_000, items=5_000, n_train=800_000, n_test=200_000, k=64, version=5,
               user_deg=("zipf", 1.0), item_deg=("zipf", 1.0), grid="int1_5",
               hyper=dict(learning_rate=0.01, decay=0.1, lam=0.05, epoch=20)),
    "c2": dict(users=71_567, items=10_681, n_train=8_000_000, n_test=2_000_000, k=128, version=1,
               user_deg=("zipf", 0.9), item_deg=("zipf", 1.1), grid="half0.5_5",
               hyper=dict(learning_rate=0.01, decay=0.1, lam=0.015, epoch=50, user_group_num=100, item_group_num=100,
                          sample_ratio=0.05, interval=2, error_threshold=20.0, thread_block_size=128)),
    "c3": dict(users=162_541, items=59_047, n_train=20_000_000, n_test=5_000_000, k=64, version=1,
               user_deg=("zipf", 1.0), item_deg=("zipf", 1.0), grid="half0.5_5",
               hyper=dict(learning_rate=0.01, decay=0.1, lam=0.015, epoch=50, user_group_num=100, item_group_num=100,
                          sample_ratio=0.05, interval=2, error_threshold=20.0, thread_block_size=128)),
    "c4": dict(users=480_189, items=17_770, n_train=100_480_507, n_test=1_408_395, k=128, version=1,
               user_deg=("lognormal", 4.5, 1.2), item_deg=("zipf", 1.2), grid="int1_5",
               hyper=dict(learning_rate=0.01, decay=0.1, lam=0.015, epoch=50, user_group_num=100, item_group_num=100,
                          sample_ratio=0.05, interval=2, error_threshold=20.0, thread_block_size=128)),
    "c5": dict(users=1_000_990, items=624_961, n_train=252_800_275, n_test=4_003_960, k=128, version=1,
               user_deg=("zipf", 1.0), item_deg=("zipf", 1.0), grid="yahoo0_100",
               hyper=dict(learning_rate=0.01, decay=0.1, lam=0.015, epoch=50, user_group_num=100, item_group_num=100,
                          sample_ratio=0.05, interval=2, error_threshold=20.0, thread_block_size=128)),
}


# -wg: the benchmark configurations quote the reference's RTX 2070 settings (2048 / 2304 warps); the
# engine's automatic choice (num_workers = 0) is used instead, see mascot_config.num_workers.
for _c in CONFIGS.values():
    _c["hyper"]["num_workers"] = 0


def scaled(cfg, factor):
    """A configuration shrunk by `factor` in every extensive quantity (same distributions)."""
    c = dict(cfg)
    for key in ("users", "items", "n_train", "n_test"):
        c[key] = max(int(cfg[key] * factor), 16)
    return c


def _weights(spec, n, rng):
    if spec[0] == "zipf":
        w = np.arange(1, n + 1, dtype=np.float64) ** (-spec[1])
    else:
        w = rng.lognormal(spec[1], spec[2], n)
    w = w / w.sum()
    # entity ids are a random relabelling of the popularity ranks
    return w[rng.permutation(n)]


def _to_grid(x, grid, rng):
    if grid == "int1_5":
        return np.clip(np.rint(3.0 + 2.5 * x), 1, 5)
    if grid == "half0.5_5":
        return np.clip(np.rint((3.0 + 2.5 * x) * 2) / 2, 0.5, 5.0)
    if grid == "yahoo0_100":
        # bimodal: a mass at 0 and a mode near 90, mostly multiples of 10; rescaled to the 1..5 range
        # the reference applies to this format (rating / 25 + 1, io_utils.h:72)
        v = 70.0 + 45.0 * x
        zero = rng.random(x.shape[0]) < 0.25
        coarse = rng.random(x.shape[0]) < 0.85
        v = np.where(coarse, np.rint(v / 10) * 10, np.rint(v))
        v = np.clip(np.where(zero, 0.0, v), 0, 100)
        return v / 25.0 + 1.0
    raise ValueError(grid)


def generate(cfg, seed=0):
    """numpy back end.  Returns (train, test) structured arrays of dtype RATING with compact ids."""
    rng = np.random.default_rng(seed)
    nu, ni = cfg["users"], cfg["items"]
    total = cfg["n_train"] + cfg["n_test"]
    if total > 0.5 * nu * ni:
        raise ValueError("requested more ratings than half of the matrix")
    cu = np.cumsum(_weights(cfg["user_deg"], nu, rng))
    ci = np.cumsum(_weights(cfg["item_deg"], ni, rng))
    keys = np.empty(0, np.uint64)
    while keys.size < total:
        want = int((total - keys.size) * 1.2) + 1024
        u = np.minimum(np.searchsorted(cu, rng.random(want)), nu - 1).astype(np.uint64)
        i = np.minimum(np.searchsorted(ci, rng.random(want)), ni - 1).astype(np.uint64)
        keys = np.unique(np.concatenate([keys, u * np.uint64(ni) + i]))
    keys = keys[rng.permutation(keys.size)[:total]]
    u = (keys // np.uint64(ni)).astype(np.uint32)
    i = (keys % np.uint64(ni)).astype(np.uint32)
    pt = (rng.standard_normal((nu, 16)) * 0.3).astype(np.float32)
    qt = (rng.standard_normal((ni, 16)) * 0.3).astype(np.float32)
    x = np.empty(total, np.float64)
    step = 1 << 22
    for b in range(0, total, step):
        sl = slice(b, min(b + step, total))
        x[sl] = np.einsum("nk,nk->n", pt[u[sl]], qt[i[sl]]) + rng.standard_normal(sl.stop - sl.start) * 0.5 / 2.5
    r = _to_grid(x, cfg["grid"], rng).astype(np.float32)
    out = np.empty(total, RATING)
    out["u"], out["i"], out["r"] = u, i, r
    train, test = out[:cfg["n_train"]], out[cfg["n_train"]:]
    # every test pair must refer to a user and an item that occur in the training set
    seen_u = np.zeros(nu, bool); seen_u[train["u"]] = True
    seen_i = np.zeros(ni, bool); seen_i[train["i"]] = True
    test = test[seen_u[test["u"]] & seen_i[test["i"]]]
    return np.ascontiguousarray(train), np.ascontiguousarray(test)


def generate_cuda(cfg, seed=0, device="cuda:0"):
    """torch/CUDA back end for the large configurations.  Returns pinned host tensors
    (train, test) of shape [n, 3] int32 holding (float bits of r, u, i) - the RATING record."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(seed)
    nu, ni = cfg["users"], cfg["items"]
    total = cfg["n_train"] + cfg["n_test"]
    rng = np.random.default_rng(seed)
    cu = torch.from_numpy(np.cumsum(_weights(cfg["user_deg"], nu, rng))).to(device)
    ci = torch.from_numpy(np.cumsum(_weights(cfg["item_deg"], ni, rng))).to(device)
    keys = torch.empty(0, dtype=torch.int64, device=device)
    while keys.numel() < total:
        want = int((total - keys.numel()) * 1.2) + 1024
        u = torch.searchsorted(cu, torch.rand(want, generator=g, device=device, dtype=torch.float64)).clamp_(max=nu - 1)
        i = torch.searchsorted(ci, torch.rand(want, generator=g, device=device, dtype=torch.float64)).clamp_(max=ni - 1)
        keys = torch.unique(torch.cat([keys, u * ni + i]))
        del u, i
    keys = keys[torch.randperm(keys.numel(), generator=g, device=device)[:total]]
    u = keys // ni
    i = keys % ni
    del keys
    pt = torch.randn(nu, 16, generator=g, device=device) * 0.3
    qt = torch.randn(ni, 16, generator=g, device=device) * 0.3
    x = torch.empty(total, device=device)
    step = 1 << 24
    for b in range(0, total, step):
        e = min(b + step, total)
        x[b:e] = (pt[u[b:e]] * qt[i[b:e]]).sum(1) + torch.randn(e - b, generator=g, device=device) * (0.5 / 2.5)
    grid = cfg["grid"]
    if grid == "int1_5":
        r = torch.clamp(torch.round(3.0 + 2.5 * x), 1, 5)
    elif grid == "half0.5_5":
        r = torch.clamp(torch.round((3.0 + 2.5 * x) * 2) / 2, 0.5, 5.0)
    else:
        v = 70.0 + 45.0 * x
        zero = torch.rand(total, generator=g, device=device) < 0.25
        coarse = torch.rand(total, generator=g, device=device) < 0.85
        v = torch.where(coarse, torch.round(v / 10) * 10, torch.round(v))
        r = torch.clamp(torch.where(zero, torch.zeros_like(v), v), 0, 100) / 25.0 + 1.0
    del x
    rec = torch.empty(total, 3, dtype=torch.int32, device=device)
    rec[:, 0] = r.to(torch.float32).view(torch.int32)
    rec[:, 1] = u.to(torch.int32)
    rec[:, 2] = i.to(torch.int32)
    nt = cfg["n_train"]
    seen_u = torch.zeros(nu, dtype=torch.bool, device=device); seen_u[u[:nt]] = True
    seen_i = torch.zeros(ni, dtype=torch.bool, device=device); seen_i[i[:nt]] = True
    keep = seen_u[u[nt:]] & seen_i[i[nt:]]
    train = torch.empty(nt, 3, dtype=torch.int32, pin_memory=True)
    train.copy_(rec[:nt])
    test_d = rec[nt:][keep]
    test = torch.empty(test_d.shape[0], 3, dtype=torch.int32, pin_memory=True)
    test.copy_(test_d)
    return train, test
