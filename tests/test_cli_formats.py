"""CPU tests of the command-line surface: the text formats of the reference (parsing rules, id
compaction, unseen-pair filtering, model file layout) and the behaviour of the tools without a GPU."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "icdm-2021_mascot_b200")
BIN = os.path.join(PKG, "bin")


@pytest.fixture(scope="session")
def io_check(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("cli") / "cli_io_check")
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(PKG, "cli"),
                           os.path.join(ROOT, "tests", "cli_io_check.cpp"), "-o", exe])
    return exe


def run(cmd):
    return subprocess.run(cmd, capture_output=True, text=True, timeout=120)


def test_tsv_parsing_compaction_and_test_filtering(io_check, tmp_path):
    d = tmp_path / "plain"
    d.mkdir()
    train = d / "train.tsv"
    test = d / "test.tsv"
    #            user item rating      (a two-token line and a blank line are skipped)
    train.write_text("10\t7\t4.5\n3\t7\t2\nbad line\n\n10\t900\t1.5 \r\n42\t5\t3\n")
    test.write_text("3\t900\t5\n10\t7\t1\n10\t7\t2\n77\t7\t3\n3\t1234\t4\n42\t5\t0.5\n")
    out = run([io_check, "parse", str(train), str(test)])
    assert out.returncode == 0, out.stderr
    lines = out.stdout.splitlines()
    assert "Missing the number of ratings : 2" in lines[0]
    assert lines[1] == "users 3 items 3 train 4 test 3 missing 2"
    T = [l.split() for l in lines if l.startswith("T ")]
    # first-seen compaction: users 10->0, 3->1, 42->2; items 7->0, 900->1, 5->2
    assert [(t[1], t[2], t[4], t[5]) for t in T] == [("0", "0", "10", "7"), ("1", "0", "3", "7"), ("0", "1", "10", "900"), ("2", "2", "42", "5")]
    assert [float(t[3]) for t in T] == [4.5, 2.0, 1.5, 3.0]
    E = [l.split()[1:] for l in lines if l.startswith("E ")]
    # ordered by (user, item) in compact ids; the repeated pair keeps its last rating
    assert E == [["0", "0", "2"], ["1", "1", "5"], ["2", "2", "0.5"]]
    assert (d / "remove_user.txt").read_text().split() == ["77"]
    assert (d / "remove_item.txt").read_text().split() == ["1234"]


def test_item_first_and_yahoo_formats(io_check, tmp_path):
    d = tmp_path / "netflix_like"
    d.mkdir()
    (d / "train.tsv").write_text("7\t10\t4\n7\t3\t2\n")          # path contains "netflix": item first
    (d / "test.tsv").write_text("7\t3\t1\n")
    out = run([io_check, "parse", str(d / "train.tsv"), str(d / "test.tsv")])
    T = [l.split() for l in out.stdout.splitlines() if l.startswith("T ")]
    assert [(t[4], t[5]) for t in T] == [("10", "7"), ("3", "7")]
    y = tmp_path / "Yahoo_like"
    y.mkdir()
    (y / "train.txt").write_text("5|2\n100\t90\n101\t0\n6|1\n100\t50\n")
    (y / "test.txt").write_text("5|1\n101\t100\n")
    out = run([io_check, "parse", str(y / "train.txt"), str(y / "test.txt")])
    lines = out.stdout.splitlines()
    assert lines[1].startswith("users 2 items 2 train 3 test 1")
    T = [l.split() for l in lines if l.startswith("T ")]
    assert [float(t[3]) for t in T] == [np.float32(90 / 25 + 1), 1.0, 3.0]      # r/25 + 1
    E = [l.split() for l in lines if l.startswith("E ")]
    assert float(E[0][3]) == 5.0


def test_model_files_round_trip(io_check, tmp_path):
    train = tmp_path / "t.tsv"
    rng = np.random.default_rng(0)
    users = rng.choice(np.arange(2, 60), 20, replace=False)
    items = rng.choice(np.arange(1, 40), 15, replace=False)
    with open(train, "w") as f:
        for u in users:
            for i in rng.choice(items, 3, replace=False):
                f.write(f"{u}\t{i}\t{rng.integers(1, 6)}\n")
    out = run([io_check, "model", str(train), str(tmp_path / "m")])
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if not l.startswith("Save")]
    n_items_used = len(set(open(train).read().split()[1::3]))
    assert lines[0] == f"orig {users.max() + 1} {max(int(x) for x in open(train).read().split()[1::3]) + 1} 64 reconst 20 {n_items_used} 64"
    err, gap = float(lines[1].split()[1]), float(lines[1].split()[3])
    assert err < 1e-5 and gap == 0.0          # 6 significant digits in the text, zero rows for id gaps
    head = open(str(tmp_path / "m") + ".txt").readline().split()
    assert len(head) == 3
    body = open(str(tmp_path / "m") + ".txt").read().split("\n")
    assert len(body[1].split()) == (users.max() + 1) * 64        # P on line 2, Q on line 3
    assert body[1].endswith(" ")


def test_binary_rating_files_and_the_converter(io_check, tmp_path):
    """convert_ratings: text -> binary -> the three text layouts, and the binary file parses to the same
    ratings as the text it came from (ids compacted in first-seen order, then stored compact)."""
    conv = os.path.join(BIN, "convert_ratings")
    if not os.path.exists(conv):
        pytest.skip("command-line tools not built")
    rng = np.random.default_rng(4)
    n = 500
    users, items = rng.integers(1, 80, n), rng.integers(1, 50, n)
    ratings = rng.choice(np.arange(0, 101, 10), n)
    y = tmp_path / "Yahoo_src"; y.mkdir()
    order = np.argsort(users, kind="stable")
    with open(y / "train.txt", "w") as f:
        for u in np.unique(users):
            rows = order[users[order] == u]
            f.write(f"{u}|{rows.size}\n")
            for j in rows:
                f.write(f"{items[j]}\t{ratings[j]}\n")
    (y / "test.txt").write_text("")
    ref = run([io_check, "parse", str(y / "train.txt"), str(y / "test.txt")]).stdout.splitlines()
    ref_T = [l for l in ref if l.startswith("T ")]
    assert len(ref_T) == n
    b = tmp_path / "ratings.bin"
    assert run([conv, str(y / "train.txt"), str(b), "bin"]).returncode == 0
    assert os.path.getsize(b) == 32 + 12 * n
    hdr = np.fromfile(b, np.uint32, 8)
    assert hdr[0] == 0x5243534d and hdr[1] == 1 and hdr[2] == n and hdr[6] == 1       # magic, version, n, compact ids
    recs = np.fromfile(b, np.dtype([("r", "<f4"), ("u", "<u4"), ("i", "<u4")]), offset=32)
    want = np.array([[float(l.split()[3]), int(l.split()[1]), int(l.split()[2])] for l in ref_T])
    assert np.array_equal(recs["u"], want[:, 1].astype(np.uint32)) and np.array_equal(recs["i"], want[:, 2].astype(np.uint32))
    assert np.array_equal(recs["r"], want[:, 0].astype(np.float32))
    # binary -> yahoo text -> parse: the same multiset of (user, item, rating) in compact ids of the binary file
    y2 = tmp_path / "Yahoo_out"; y2.mkdir()
    assert run([conv, str(b), str(y2 / "train.txt"), "yahoo"]).returncode == 0
    back = run([io_check, "parse", str(y2 / "train.txt"), str(y / "test.txt")]).stdout.splitlines()
    trip = lambda lines: sorted((int(l.split()[4]), int(l.split()[5]), float(l.split()[3])) for l in lines if l.startswith("T "))
    assert trip(back) == sorted((int(u), int(i), float(r)) for r, u, i in want)
    # tsv and item-first layouts
    t = tmp_path / "plain"; t.mkdir()
    assert run([conv, str(b), str(t / "train.tsv"), "tsv"]).returncode == 0
    rows = [l.split("\t") for l in open(t / "train.tsv").read().splitlines()]
    assert len(rows) == n and [int(r[0]) for r in rows] == recs["u"].tolist()
    assert np.array_equal(np.array([r[2] for r in rows], np.float32), recs["r"]), "ratings survive the text form exactly"
    nf = tmp_path / "netflix_out"; nf.mkdir()
    assert run([conv, str(b), str(nf / "train.tsv"), "item_first"]).returncode == 0
    rows = [l.split("\t") for l in open(nf / "train.tsv").read().splitlines()]
    assert [int(r[0]) for r in rows] == recs["i"].tolist() and [int(r[1]) for r in rows] == recs["u"].tolist()


def test_binary_model_round_trip(io_check, tmp_path):
    out = run([io_check, "binmodel", str(tmp_path / "m.bin")])
    assert out.returncode == 0 and "binmodel identical" in out.stdout


def test_tools_fail_loudly_without_a_gpu(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    exe = os.path.join(BIN, "quantized_mf")
    if not os.path.exists(exe):
        pytest.skip("command-line tools not built")
    (tmp_path / "train.tsv").write_text("1\t2\t3\n2\t2\t4\n")
    (tmp_path / "test.tsv").write_text("1\t2\t5\n")
    out = run([exe, "-i", str(tmp_path / "train.tsv"), "-y", str(tmp_path / "test.tsv"), "-v", "5", "-k", "64", "-l", "2"])
    assert out.returncode == 1
    assert "Latent features             : 64" in out.stdout and "The number of nonzeros      : 2" in out.stdout
    assert "no CUDA device" in out.stderr
    out = run([exe, "-i", str(tmp_path / "nope.tsv")])
    assert out.returncode == 0 and "doesn't exist!" in out.stdout
