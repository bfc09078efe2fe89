"""GPU test of mascot_rmse_device_noalloc, the evaluation entry point for callers that may not
allocate device memory when they call (a host program whose memory pool owns the whole GPU, a
serving loop that cannot take cudaMalloc's device-wide synchronisation, a fixed memory budget).

It is called through the C ABI on device buffers and must return exactly what the allocating entry
point mascot_rmse_device returns - the comparison is bit-exact, like every other RMSE comparison in
this suite - on two calls in a row, the second on a smaller test set so that stale partials of the
first call sit in the shared scratch array.  Collected last on purpose (file name)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_RATINGS = 65536 * 512


def _device_problem(torch, k, n_users, n_items, n_test, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    P = torch.randn(n_users, k, generator=g, device="cuda") * 0.2
    Q = torch.randn(n_items, k, generator=g, device="cuda") * 0.2
    rec = torch.empty(n_test, 3, dtype=torch.int32, device="cuda")
    r = torch.randint(1, 6, (n_test,), generator=g, device="cuda").to(torch.float32)
    rec[:, 0] = r.view(torch.int32)
    rec[:, 1] = torch.randint(0, n_users, (n_test,), generator=g, device="cuda").to(torch.int32)
    rec[:, 2] = torch.randint(0, n_items, (n_test,), generator=g, device="cuda").to(torch.int32)
    torch.cuda.synchronize()
    return P, Q, rec


def _call(lib, name, P, Q, k, rec, n):
    out = C.c_double(-1.0)
    rc = getattr(lib, name)(C.c_void_p(P.data_ptr()), C.c_void_p(Q.data_ptr()), C.c_uint32(k),
                            C.c_void_p(rec.data_ptr()), C.c_uint64(n), C.byref(out))
    return rc, out.value


@pytest.mark.parametrize("k", (128, 64))
def test_noalloc_entry_point_matches_the_allocating_one_twice_in_a_row(mascot, k):
    import torch
    lib = mascot.load()
    torch.cuda.set_device(0)
    P, Q, rec = _device_problem(torch, k, 5000, 3000, 300_000, seed=k)
    for n in (300_000, 70_001):          # second call: fewer blocks than the first left behind
        rc_a, want = _call(lib, "mascot_rmse_device", P, Q, k, rec, n)
        rc_b, got = _call(lib, "mascot_rmse_device_noalloc", P, Q, k, rec, n)
        assert rc_a == 0 and rc_b == 0, lib.mascot_last_error(None)
        assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32), (n, got, want)
        # and both agree with a float64 recomputation to 1e-5 relative
        u, i = rec[:n, 1].long(), rec[:n, 2].long()
        pred = (P[u].double() * Q[i].double()).sum(1)
        ref = torch.sqrt(((rec[:n, 0].view(torch.float32).double() - pred) ** 2).mean()).item()
        assert abs(got - ref) <= 1e-5 * ref


def test_noalloc_entry_point_rejects_sizes_beyond_its_scratch(mascot):
    import torch
    lib = mascot.load()
    torch.cuda.set_device(0)
    P, Q, rec = _device_problem(torch, 64, 64, 64, 1024, seed=1)
    rc, _ = _call(lib, "mascot_rmse_device_noalloc", P, Q, 64, rec, MAX_RATINGS + 1)
    assert rc == mascot.ERR_BAD_ARG
    assert b"at most 33554432" in lib.mascot_last_error(None)
    rc, _ = _call(lib, "mascot_rmse_device_noalloc", P, Q, 96, rec, 1024)
    assert rc == mascot.ERR_BAD_ARG
    rc, v = _call(lib, "mascot_rmse_device_noalloc", P, Q, 64, rec, 1024)
    assert rc == 0 and np.isfinite(v)
