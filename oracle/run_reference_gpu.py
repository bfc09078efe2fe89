"""Run the reference's own CUDA build and this engine on the same seeded synthetic files, on the GPU
box, and report both: update-kernel time per epoch, updates/s and the test-RMSE trajectory.

TEST / MEASUREMENT INFRASTRUCTURE.  Needs oracle/_ref/quantized_mf (built from the reference tree by
`make -C oracle ref`; the binary travels, the reference sources do not) and a GPU.

    python oracle/run_reference_gpu.py --workload c2 --epochs 20 --wg 2048,9472 --out ref_c2.json

The reference sizes the dynamic shared memory of its MASCOT kernel 8 bytes short when a side has
more than 62 groups; that stays inside the allocation unless the requested size is within 8 bytes of
a multiple of the 128-byte allocation granule.  The group counts are computed here first (same
grouping algorithm) and the requested group number is lowered until the launch is safe by that rule.
"""
import argparse
import importlib.util
import json
import os
import re
import subprocess
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
PKG = os.path.join(ROOT, "icdm-2021_mascot_b200")
sys.path.insert(0, HERE)


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def write_tsv(path, recs):
    import pyarrow as pa
    import pyarrow.csv as pc
    t = pa.table({"u": recs["u"].astype(np.int64), "i": recs["i"].astype(np.int64), "r": recs["r"].astype(np.float64)})
    pc.write_csv(t, path, write_options=pc.WriteOptions(include_header=False, delimiter="\t", quoting_style="none"))


def smem_request_is_safe(ug, ig):
    if ug <= 62 and ig <= 62:
        return True
    size = 12 * (ug + ig) + 4 * max(ug - 62, 0) + 4 * max(ig - 62, 0) + (ug + ig)
    over = 4 * (ug > 62) + 4 * (ig > 62)
    room = (-size) % 128
    return room >= over


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--wg", default="2048")
    ap.add_argument("--seed", type=int, default=4)
    ap.add_argument("--out", default="reference_gpu.json")
    ap.add_argument("--dir", default=os.path.join(HERE, "_ref", "data"), help="where the rating files are written (git-ignored)")
    ap.add_argument("--skip-reference", action="store_true")
    ap.add_argument("--workers", default="0", help="comma list: worker counts (-wg) of this engine to try (0 = the configuration's)")
    args = ap.parse_args()

    import oracle as O
    S = _load("mascot_synth", os.path.join(PKG, "synth.py"))
    M = _load("mascot_binding", os.path.join(PKG, "mascot.py"))
    cfg = S.CONFIGS[args.workload]
    if args.scale != 1.0:
        cfg = S.scaled(cfg, args.scale)
    hy = dict(cfg["hyper"]); hy["epoch"] = args.epochs
    t0 = time.time()
    train_t, test_t = S.generate_cuda(cfg, seed=args.seed)
    train = train_t.numpy().view(np.uint32).reshape(-1, 3).view(M.RATING).reshape(-1)
    test = test_t.numpy().view(np.uint32).reshape(-1, 3).view(M.RATING).reshape(-1)
    gen_s = time.time() - t0

    result = {"workload": args.workload, "scale": args.scale, "users": cfg["users"], "items": cfg["items"],
              "n_train": int(train.size), "n_test": int(test.size), "epochs": args.epochs, "k": cfg["k"],
              "version": cfg["version"], "gen_s": gen_s, "reference": [], "ours": None}

    ug_req, ig_req = hy.get("user_group_num", 10), hy.get("item_group_num", 10)
    if cfg["version"] == 1:
        _, _, cnt_u = O.degree_sort(train["u"], cfg["users"])
        _, _, cnt_i = O.degree_sort(train["i"], cfg["items"])
        while True:
            ug, ig = len(O.grouping(cnt_u, ug_req)[0]), len(O.grouping(cnt_i, ig_req)[0])
            if smem_request_is_safe(ug, ig):
                break
            ug_req -= 1
        hy["user_group_num"], hy["item_group_num"] = ug_req, ig_req
        result["groups"] = {"requested": [ug_req, ig_req], "actual": [ug, ig]}

    # ---- this engine ----
    runs = []
    for gb in [int(x) for x in args.workers.split(",")]:
        hw = dict(hy)
        if gb:
            hw["num_workers"] = gb
        ecfg = M.default_config(version=cfg["version"], k=cfg["k"], seed=args.seed, **hw)
        eng = M.Engine(ecfg)
        eng.set_ratings(train, test, cfg["users"], cfg["items"])
        eng.init_factors()
        ours = {"workers": gb, "rmse": [], "kernel_ms": [], "total_ms": [], "promoted": []}
        for e in range(args.epochs):
            st = eng.train_epoch(e)
            ours["rmse"].append(eng.eval_rmse()); ours["kernel_ms"].append(st.kernel_ms); ours["total_ms"].append(st.total_ms)
            ours["promoted"].append([st.promoted_user_groups, st.promoted_item_groups])
        ours["updates_per_epoch"] = int(train.size)
        ours["updates_per_s"] = train.size * args.epochs / (sum(ours["total_ms"]) * 1e-3)
        ours["final_precisions_fp32_groups"] = [int(eng.group_info(0)[1].sum()), int(eng.group_info(1)[1].sum())]
        eng.close()
        runs.append(ours)
        print("ours workers", gb, st.workers, "updates/s %.3g" % ours["updates_per_s"], "rmse", [round(x, 4) for x in ours["rmse"][::3]], flush=True)
    ours = runs[0]
    result["ours"] = ours
    result["ours_all"] = runs

    # ---- the reference's CUDA build on the same files ----
    exe = os.path.join(HERE, "_ref", "quantized_mf")
    if not args.skip_reference and os.path.exists(exe):
        os.makedirs(args.dir, exist_ok=True)
        tr, te = os.path.join(args.dir, "ratings_train.tsv"), os.path.join(args.dir, "ratings_test.tsv")
        t0 = time.time()
        write_tsv(tr, train); write_tsv(te, test)
        result["write_s"] = time.time() - t0
        for wg in [int(w) for w in args.wg.split(",")]:
            cmd = [exe, "-i", tr, "-y", te, "-k", str(cfg["k"]), "-l", str(args.epochs), "-a", str(hy["learning_rate"]),
                   "-d", str(hy["decay"]), "-b", str(hy["lam"]), "-wg", str(wg), "-bl", "128", "-v", str(cfg["version"]),
                   "-ug", str(hy.get("user_group_num", 10)), "-ig", str(hy.get("item_group_num", 10)),
                   "-s", str(hy.get("sample_ratio", 0.01)), "-it", str(hy.get("interval", 1)),
                   "-e", str(hy.get("error_threshold", 0.001))]
            t0 = time.time()
            p = subprocess.run(cmd, capture_output=True, text=True, timeout=3000)
            wall = time.time() - t0
            out = p.stdout
            rm = [float(m.group(3)) for m in re.finditer(r"^(\d+) ([0-9.eE+-]+) ([0-9.eE+-]+|nan|-nan|inf)\s*$", out, flags=re.M)]
            per_epoch = re.search(r"(?:Parameters update per epoch|Execution time\(avg per epoch\))\s*:\s*([0-9.eE+]+)", out)
            upd_count = int(np.ceil(train.size / (wg * 128)))
            updates = wg * upd_count * 128
            entry = {"wg": wg, "rc": p.returncode, "wall_s": wall, "rmse": rm,
                     "kernel_us_per_epoch": float(per_epoch.group(1)) if per_epoch else None,
                     "updates_per_epoch": updates, "stderr_tail": p.stderr[-300:]}
            if entry["kernel_us_per_epoch"]:
                entry["updates_per_s"] = updates / (entry["kernel_us_per_epoch"] * 1e-6)
            result["reference"].append(entry)
            with open(os.path.join(os.path.dirname(args.out) or ".", f"reference_stdout_wg{wg}.txt"), "w") as f:
                f.write(out[-20000:])
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    with open(args.out, "w") as f:
        json.dump(result, f, indent=1)
    brief = {"ours_updates_per_s": ours["updates_per_s"], "ours_final_rmse": ours["rmse"][-1],
             "reference": [{k: e.get(k) for k in ("wg", "rc", "updates_per_s", "kernel_us_per_epoch", "wall_s")} |
                           {"final_rmse": (e["rmse"][-1] if e["rmse"] else None)} for e in result["reference"]]}
    print(json.dumps(brief))


if __name__ == "__main__":
    main()
