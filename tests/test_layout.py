"""CPU tests of the row layout and the seeded permutation (icdm-2021_mascot_b200/csrc/layout.cuh), which
host and device code share: compiled here with g++ and checked against the properties the update
kernel relies on."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "icdm-2021_mascot_b200", "csrc")


@pytest.fixture(scope="session")
def layout_check(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("layout") / "layout_check")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-I", CSRC, os.path.join(ROOT, "tests", "layout_check.cpp"), "-o", exe])
    return exe


def tables(exe):
    out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split("\n")
    res, cur = {}, None
    for line in out:
        if line.startswith("K "):
            cur = int(line.split()[1]); res[cur] = []
        elif line:
            res[cur].append(tuple(int(x) for x in line.split()))
    return res


def test_layout_is_a_bijection_and_its_inverse(layout_check):
    for K, rows in tables(layout_check).items():
        logical = [l for l, _ in rows]
        assert sorted(logical) == list(range(K))
        assert [p for _, p in rows] == list(range(K)), "phys_of_logical inverts logical_of_phys"


def test_a_lane_holds_the_operands_of_whole_reference_lanes(layout_check):
    """Lane m of a worker owns physical elements 8m..8m+7.  The reference gives lane l the elements
    l, l+32[, l+64, l+96] and folds lanes with shfl_down 16, 8, 4, 2, 1: the eight elements must be
    the complete operand sets of reference lanes m and m+16 (k=128) or m, m+16, m+8, m+24 (k=64), stored
    as the pairs (e0,e4) (e1,e5) (e2,e6) (e3,e7)."""
    t = tables(layout_check)
    for m in range(16):
        e = [l for l, _ in t[128][8 * m:8 * m + 8]]
        lane_a = [m, m + 32, m + 64, m + 96]                 # slots 0..3 of reference lane m
        lane_b = [m + 16, m + 48, m + 80, m + 112]           # ... of reference lane m+16
        assert e == [lane_a[0], lane_b[0], lane_a[1], lane_b[1], lane_a[2], lane_b[2], lane_a[3], lane_b[3]]
    for m in range(8):
        e = [l for l, _ in t[64][8 * m:8 * m + 8]]
        l0, l1, l2, l3 = [m, m + 32], [m + 16, m + 48], [m + 8, m + 40], [m + 24, m + 56]   # lanes m, m+16, m+8, m+24
        # e0,e1 = lane m; e2,e3 = lane m+16; e4,e5 = lane m+8; e6,e7 = lane m+24; stored e0 e4 e1 e5 e2 e6 e3 e7
        assert e == [l0[0], l2[0], l0[1], l2[1], l1[0], l3[0], l1[1], l3[1]]


@pytest.mark.parametrize("n,seed", [(1, 3), (2, 3), (17, 0), (1000, 12345), (4097, 99)])
def test_seeded_permutation_is_a_bijection(layout_check, n, seed):
    out = subprocess.run([layout_check, "p", str(n), str(seed)], capture_output=True, text=True, check=True).stdout.split()
    v = np.array([int(x) for x in out])
    assert v.size == n and np.array_equal(np.sort(v), np.arange(n))
    if n > 100:
        assert (v != np.arange(n)).mean() > 0.9, "not the identity"
        other = subprocess.run([layout_check, "p", str(n), str(seed + 1)], capture_output=True, text=True, check=True).stdout.split()
        assert (v != np.array([int(x) for x in other])).mean() > 0.9, "depends on the seed"


def test_launch_cache_raises_the_shared_memory_limit_once_and_never_lowers_it(tmp_path):
    """csrc/launch_cache.h: a full-grid launch, then a single-block launch that needs little shared
    memory, then the full-grid shape again (the order that used to lose the opt-in): the limit is set
    once per device, to the kernel's largest request, and the occupancy answer is asked once per shape."""
    exe = str(tmp_path / "launch_cache_check")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-I", CSRC, os.path.join(ROOT, "tests", "launch_cache_check.cpp"), "-o", exe])
    seq = ["0:224:50176", "0:32:7168", "0:224:50176", "1:224:50176", "0:32:7168"]
    out = subprocess.run([exe, "57344", "0"] + seq, capture_output=True, text=True, check=True).stdout.strip().split("\n")
    raises = [l for l in out if l.startswith("raise")]
    assert raises == ["raise dev=0 bytes=57344", "raise dev=1 bytes=57344"]
    queries = [l for l in out if l.startswith("query")]
    assert queries == ["query dev=0 block=224 smem=50176", "query dev=0 block=32 smem=7168", "query dev=1 block=224 smem=50176"]
    launches = [l for l in out if l.startswith("launch")]
    assert len(launches) == 5 and all(" rc=0 " in l for l in launches)
    assert launches[0].split("fit=")[1] == launches[2].split("fit=")[1]
    # a failing raise is reported, and tried again by the next launch
    out = subprocess.run([exe, "57344", "7", "0:224:50176", "0:224:50176"], capture_output=True, text=True, check=True).stdout
    assert out.count("raise dev=0") == 2 and out.count("rc=7") == 2


def test_bounded_wait_returns_ok_error_or_timeout(tmp_path):
    """csrc/bounded_wait.h, the wait behind every cross-rank dependency of the sharded path: finished
    work ends it with 0, a failing poll with that failure, and work that never finishes with
    MASCOT_ERR_TIMEOUT (-6) once the limit has passed - never later than a little after the limit."""
    exe = str(tmp_path / "bounded_wait_check")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-I", CSRC, os.path.join(ROOT, "tests", "bounded_wait_check.cpp"), "-o", exe])
    run = lambda *a: subprocess.run([exe] + [str(x) for x in a], capture_output=True, text=True, check=True).stdout.split()
    rc, ms, polls = run(5, 2000, 0)
    assert rc == "0" and int(polls) == 6 and float(ms) < 500
    rc, ms, polls = run(-1, 200, 0)                  # never ready
    assert rc == "-6" and 200 <= float(ms) < 1500
    rc, ms, polls = run(-1, 5000, -8)                # the poll reports a communication failure
    assert rc == "-8" and int(polls) == 3 and float(ms) < 1000


def test_fast_rounding_and_power_of_two_reciprocal_are_exact(tmp_path):
    """The fixed-point trainers' kernels replace roundf by trunc(x + copysign(largest float below 1/2, x)) and
    1 / (power of two) by the mirrored exponent; the host restatement checks the first on all 2^32 float
    patterns and the second on every power of two it applies to."""
    exe = str(tmp_path / "round_check")
    subprocess.check_call(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", os.path.join(ROOT, "tests", "round_check.c"), "-o", exe, "-lm"])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout


def test_integer_ceil_log2_equals_the_double_precision_formula(tmp_path):
    """The AFP trainer's kernel computes ceil((float)log2((double)x)) - the exponent of its fixed-point scale -
    from the bits of x; the host restatement of that shortcut is compared with the formula on every positive
    finite float."""
    exe = str(tmp_path / "ceil_log2_check")
    subprocess.check_call(["gcc", "-O2", "-fopenmp", os.path.join(ROOT, "tests", "ceil_log2_check.c"), "-o", exe, "-lm"])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout
