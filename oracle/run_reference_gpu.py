"""Run the reference's own CUDA build and this engine on the same seeded synthetic ratings, on the GPU
box, and report both: update-kernel time per epoch, updates/s and the test-RMSE trajectory, for one or
several training variants (-v).

TEST / MEASUREMENT INFRASTRUCTURE.  Needs oracle/_ref/quantized_mf (built from the reference tree by
`make -C oracle ref`; the binary travels, the reference sources do not), the engine's command-line tools
(icdm-2021_mascot_b200/bin) and a GPU.

    python oracle/run_reference_gpu.py --workload c2 --epochs 20 --wg 2048,9472 --out ref_c2.json
    python oracle/run_reference_gpu.py --workload c5 --scale 0.5 --variants 1,4,3,2 --out ref_c5.json

The ratings are generated once, written as the binary rating file of the command-line tools and converted
(bin/convert_ratings) to the text layout the reference reads: plain TSV, or - for the 252M-rating
configuration, whose 0..100 ratings both programs rescale to r/25 + 1 when the path contains "Yahoo" - the
"<user>|<count>" block format (io_utils.h:49-79).  The first variant runs alone, so that its kernel times
are clean; further variants of the reference run side by side (their input parsing, minutes of one host
core each, dominates; their kernel times then overlap and are marked as such).

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


def smem_request_is_safe(ug, ig):
    if ug <= 62 and ig <= 62:
        return True
    size = 12 * (ug + ig) + 4 * max(ug - 62, 0) + 4 * max(ig - 62, 0) + (ug + ig)
    over = 4 * (ug > 62) + 4 * (ig > 62)
    room = (-size) % 128
    return room >= over


def reference_command(exe, tr, te, cfg, hy, version, wg, epochs):
    return [exe, "-i", tr, "-y", te, "-k", str(cfg["k"]), "-l", str(epochs), "-a", str(hy["learning_rate"]),
            "-d", str(hy["decay"]), "-b", str(hy["lam"]), "-wg", str(wg), "-bl", "128", "-v", str(version),
            "-ug", str(hy.get("user_group_num", 10)), "-ig", str(hy.get("item_group_num", 10)),
            "-s", str(hy.get("sample_ratio", 0.01)), "-it", str(hy.get("interval", 1)),
            "-e", str(hy.get("error_threshold", 0.001))]


def parse_reference(out, n_train, wg):
    rm = [float(m.group(3)) for m in re.finditer(r"(?:^|(?<= ))(\d+) ([0-9.eE+-]+) ([0-9.eE+-]+|nan|-nan|inf)\s*$", out, flags=re.M)]
    per_epoch = re.search(r"(?:Parameters update per epoch|Execution time\(avg per epoch\))\s*:\s*([0-9.eE+]+)", out)
    updates = wg * int(np.ceil(n_train / (wg * 128))) * 128
    entry = {"rmse": rm, "kernel_us_per_epoch": float(per_epoch.group(1)) if per_epoch else None, "updates_per_epoch": updates}
    if entry["kernel_us_per_epoch"]:
        entry["updates_per_s"] = updates / (entry["kernel_us_per_epoch"] * 1e-6)
    return entry


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--epochs", type=int, default=0, help="0 = the configuration's")
    ap.add_argument("--wg", default="2048", help="comma list of -wg values for the reference (first variant only)")
    ap.add_argument("--variants", default="", help="comma list of -v values; default: the configuration's")
    ap.add_argument("--seed", type=int, default=4)
    ap.add_argument("--out", default="reference_gpu.json")
    ap.add_argument("--dir", default="", help="where the rating files are written (default: a Yahoo-named folder under oracle/_ref/data)")
    ap.add_argument("--skip-reference", action="store_true")
    ap.add_argument("--workers", default="0", help="comma list: worker counts (-wg) of this engine to try (0 = automatic)")
    args = ap.parse_args()

    import oracle as O
    S = _load("mascot_synth", os.path.join(PKG, "synth.py"))
    M = _load("mascot_binding", os.path.join(PKG, "mascot.py"))
    cfg = S.CONFIGS[args.workload]
    if args.scale != 1.0:
        cfg = S.scaled(cfg, args.scale)
    yahoo = cfg["grid"] == "yahoo0_100"
    hy = dict(cfg["hyper"])
    epochs = args.epochs or int(hy["epoch"])
    hy["epoch"] = epochs
    variants = [int(v) for v in args.variants.split(",")] if args.variants else [cfg["version"]]
    t0 = time.time()
    train_t, test_t = S.generate_cuda(cfg, seed=args.seed)
    train = train_t.numpy().view(np.uint32).reshape(-1, 3).view(M.RATING).reshape(-1)
    test = test_t.numpy().view(np.uint32).reshape(-1, 3).view(M.RATING).reshape(-1)
    gen_s = time.time() - t0

    result = {"workload": args.workload, "scale": args.scale, "users": cfg["users"], "items": cfg["items"],
              "n_train": int(train.size), "n_test": int(test.size), "epochs": epochs, "k": cfg["k"],
              "variants": variants, "gen_s": gen_s, "factor_bytes_fp16": int((cfg["users"] + cfg["items"]) * cfg["k"] * 2),
              "format": "yahoo blocks" if yahoo else "tsv", "reference": [], "ours": []}

    ug_req, ig_req = hy.get("user_group_num", 10), hy.get("item_group_num", 10)
    if 1 in variants or 6 in variants:
        _, _, cnt_u = O.degree_sort(train["u"], cfg["users"])
        _, _, cnt_i = O.degree_sort(train["i"], cfg["items"])
        while True:
            ug, ig = len(O.grouping(cnt_u, ug_req)[0]), len(O.grouping(cnt_i, ig_req)[0])
            if smem_request_is_safe(ug, ig):
                break
            ug_req -= 1
        hy["user_group_num"], hy["item_group_num"] = ug_req, ig_req
        result["groups"] = {"requested": [ug_req, ig_req], "actual": [ug, ig]}

    # ---- this engine, every variant ----
    for version in variants:
        for gb in [int(x) for x in args.workers.split(",")]:
            hw = dict(hy)
            if gb:
                hw["num_workers"] = gb
            ecfg = M.default_config(version=version, k=cfg["k"], seed=args.seed, is_yahoo=1 if yahoo else 0, **hw)
            eng = M.Engine(ecfg)
            eng.set_ratings(train, test, cfg["users"], cfg["items"])
            eng.init_factors()
            ours = {"version": version, "workers_requested": gb, "rmse": [], "kernel_ms": [], "total_ms": [], "promoted": [], "pass_bits": []}
            st = None
            for e in range(epochs):
                st = eng.train_epoch(e)
                ours["rmse"].append(eng.eval_rmse()); ours["kernel_ms"].append(st.kernel_ms); ours["total_ms"].append(st.total_ms)
                ours["promoted"].append([st.promoted_user_groups, st.promoted_item_groups]); ours["pass_bits"].append(st.pass_bits)
            ours["workers"] = int(st.workers)
            ours["updates_per_epoch"] = int(train.size)
            ours["updates_per_s"] = train.size * epochs / (sum(ours["total_ms"]) * 1e-3)
            ours["final_rmse"] = ours["rmse"][-1]
            ours["final_precisions_fp32_groups"] = [int(eng.group_info(0)[1].sum()), int(eng.group_info(1)[1].sum())]
            eng.close()
            result["ours"].append(ours)
            print("ours -v", version, "workers", ours["workers"], "updates/s %.3g" % ours["updates_per_s"], "rmse",
                  [round(x, 4) for x in ours["rmse"][::max(epochs // 8, 1)]], round(ours["final_rmse"], 5), flush=True)

    # ---- the reference's CUDA build on the same ratings ----
    exe = os.path.join(HERE, "_ref", "quantized_mf")
    conv = os.path.join(PKG, "bin", "convert_ratings")
    if not args.skip_reference and os.path.exists(exe) and os.path.exists(conv):
        ddir = args.dir or os.path.join(HERE, "_ref", "data", "Yahoo_like" if yahoo else "plain")
        os.makedirs(ddir, exist_ok=True)
        t0 = time.time()
        files = {}
        for name, recs in (("train", train), ("test", test)):
            b = os.path.join(ddir, f"ratings_{name}.bin")
            txt = os.path.join(ddir, f"ratings_{name}.txt")
            M.write_binary_ratings(b, recs, cfg["users"], cfg["items"])
            subprocess.check_call([conv, b, txt, "yahoo" if yahoo else "tsv"])
            os.remove(b)
            files[name] = txt
        result["write_s"] = time.time() - t0
        result["train_file_bytes"] = os.path.getsize(files["train"])
        wgs = [int(w) for w in args.wg.split(",")]
        out_dir = os.path.dirname(args.out) or "."
        os.makedirs(out_dir, exist_ok=True)

        def finish(version, wg, p, wall, shared):
            entry = {"version": version, "wg": wg, "rc": p.returncode, "wall_s": wall, "gpu_shared_with_other_runs": shared,
                     "stderr_tail": p.stderr[-300:]}
            entry.update(parse_reference(p.stdout, train.size, wg))
            entry["final_rmse"] = entry["rmse"][-1] if entry["rmse"] else None
            result["reference"].append(entry)
            with open(os.path.join(out_dir, f"reference_stdout_{args.workload}_v{version}_wg{wg}.txt"), "w") as f:
                f.write(p.stdout[-20000:])
            print("reference -v", version, "wg", wg, "rc", p.returncode, "updates/s", entry.get("updates_per_s"), "final rmse", entry["final_rmse"],
                  "wall %.0f s" % wall, flush=True)

        # the first variant alone (clean kernel times), at every requested -wg
        for wg in wgs:
            t0 = time.time()
            p = subprocess.run(reference_command(exe, files["train"], files["test"], cfg, hy, variants[0], wg, epochs), capture_output=True, text=True, timeout=3000)
            finish(variants[0], wg, p, time.time() - t0, False)
        # the other variants side by side
        rest = variants[1:]
        t0 = time.time()
        procs = [(v, subprocess.Popen(reference_command(exe, files["train"], files["test"], cfg, hy, v, wgs[0], epochs),
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)) for v in rest]
        for v, pr in procs:
            so, se = pr.communicate(timeout=3000)
            finish(v, wgs[0], subprocess.CompletedProcess(pr.args, pr.returncode, so, se), time.time() - t0, len(rest) > 1)
        for f in files.values():
            os.remove(f)
    # ---- summary: final RMSE of both builds per variant ----
    table = []
    for o in result["ours"]:
        refs = [r for r in result["reference"] if r["version"] == o["version"] and r["final_rmse"] is not None]
        if refs:
            r = refs[0]
            table.append({"version": o["version"], "ours_final_rmse": o["final_rmse"], "reference_final_rmse": r["final_rmse"],
                          "relative_difference": (o["final_rmse"] - r["final_rmse"]) / r["final_rmse"],
                          "ours_updates_per_s": o["updates_per_s"], "reference_updates_per_s": r.get("updates_per_s")})
    result["comparison"] = table
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    with open(args.out, "w") as f:
        json.dump(result, f, indent=1)
    print(json.dumps(table))


if __name__ == "__main__":
    main()
