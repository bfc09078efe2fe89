"""Benchmark of the MASCOT training hot path: rating updates per second at k=128.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4|c5|c1|c2|c3]

A "step" is one training epoch = one pass of the update kernels over the whole rating stream of the
workload (default c4: 480,189 x 17,770, 100,480,507 ratings, MASCOT variant, k=128, with its g-switching
check epochs; c5: 1,000,990 x 624,961, 252,800,275 ratings, the configuration whose factors exceed L2).
Synthetic, seeded data with the shapes and distributions of the benchmark configurations.

`value`  : updates/s with the rating stream resident in HBM, timed with CUDA events on the engine's
           stream over exactly K epochs (update kernels + statistics + precision switching).  The line
           also gives the value of each precision phase (before / after the first promotion).
`e2e`    : the same metric through the C ABI from HOST buffers: every step copies the step's rating
           stream from pinned host memory to the device, trains the epoch and reads the test RMSE back.
N > 1    : one process per GPU; the whole multi-GPU epoch (block schedule, NCCL hand-overs, statistics
           all-reduce) runs inside libmascot (mascot_shard_*); torch.distributed only carries the 128-byte
           group id and the barriers of the measurement.
`--impl reference` times the host-core loop of the same update rule (oracle/host_loop.cpp; the reference
is CUDA-only and has no CPU path) on all host cores, on a bounded sample of the same workload.
"""
import argparse
import importlib.util
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "icdm-2021_mascot_b200")


def _load(name, path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of the given GPUs while the timed region runs.

    Reads through NVML inside this process (a query takes microseconds); falls back to polling
    `nvidia-smi` when the NVML binding is missing.  Read-only: no setting of any GPU is touched."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    # bits of nvmlDeviceGetCurrentClocksEventReasons
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, indices):
        super().__init__(daemon=True)
        self.indices = [indices] if isinstance(indices, int) else list(indices)
        self.mhz, self.max_mhz, self.reasons = [], None, set()
        self.count = 0
        self.stop_flag = threading.Event()

    def _run_nvml(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            hs = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in self.indices]
            self.max_mhz = float(max(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM) for h in hs))
            reasons_of = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self.stop_flag.is_set():
                for h in hs:
                    self.mhz.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    mask = int(reasons_of(h))
                    self.reasons.update(n for n, bit in self.BITS.items() if mask & bit)
                self.count += 1
                self.stop_flag.wait(0.05)
        finally:
            pynvml.nvmlShutdown()

    def _run_smi(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", ",".join(str(i) for i in self.indices), f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                for row in out.strip().splitlines():
                    parts = [p.strip() for p in row.split(",")]
                    if len(parts) >= 6 and parts[0].replace(".", "").isdigit():
                        self.mhz.append(float(parts[0])); self.max_mhz = float(parts[1])
                        self.reasons.update(n for j, n in enumerate(names) if parts[2 + j].lower().startswith("active"))
                self.count += 1
            except Exception:
                pass
            self.stop_flag.wait(0.5)

    def run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def summary(self):
        if not self.mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        order = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        return {"sm_mhz": statistics.median(self.mhz), "sm_max_mhz": self.max_mhz,
                "reasons": [n for n in order if n in self.reasons], "samples": self.count, "gpus": self.indices}


# The reference's own CUDA build (oracle/_ref/quantized_mf, sm_100) on the same synthetic data and one
# B200, measured earlier with oracle/run_reference_gpu.py at full size.  A FALLBACK, labelled as such:
# the bench measures the build itself on a scaled copy of the workload when the binary is present.
REFERENCE_CUDA_BUILD_EARLIER_RUNS = {
    "c1": {"updates_per_s": 2.90e9, "wg": 2048, "final_rmse": 1.03972, "epochs": 20},
    "c2": {"updates_per_s": 1.53e9, "wg": 2048, "final_rmse": 0.618434, "epochs": 50},
    "c3": {"updates_per_s": 2.55e9, "wg": 2304, "final_rmse": 0.638323, "epochs": 50},
    "c4": {"updates_per_s": 1.559e9, "wg": 2048, "final_rmse": 0.601266, "epochs": 50},
}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def host_threads():
    """Cores this process may use.  torch.distributed.run exports OMP_NUM_THREADS=1, which says nothing
    about the machine; the affinity mask does."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def engine_config(M, cfg, **extra):
    hy = dict(cfg["hyper"])
    kw = dict(version=cfg["version"], k=cfg["k"], **hy)
    kw.update(extra)
    return M.default_config(**kw)


def traffic_table(workload):
    """Per-update byte counts of the dominant kernel from the committed ncu summaries (profiles/)."""
    path = os.path.join(ROOT, "profiles", "train_kernel_traffic.json")
    try:
        data = json.load(open(path))
        return data.get(workload) if isinstance(data.get(workload), dict) else (data if data.get("workload") == workload else None)
    except Exception:
        return None


# ---------------------------------------------------------------------------------------------
# host-core baseline
# ---------------------------------------------------------------------------------------------
def host_loop_model(S, cfg, seed, n_sample):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as O
    small = dict(cfg, n_train=n_sample, n_test=1000)
    train, _ = S.generate(small, seed=seed)          # same shapes and distributions; only the count is bounded
    k = cfg["k"]
    rng = np.random.default_rng(seed)
    P = (rng.standard_normal((cfg["users"], k)) * 0.01).astype(np.float32)
    Q = (rng.standard_normal((cfg["items"], k)) * 0.01).astype(np.float32)
    model = O.HostLoopModel(k, P, Q, half=(cfg["version"] == 1))
    return O, model, train


def run_reference(args, S, cfg):
    """CPU arm: the host-core loop of the update rule (a port: the reference has no CPU implementation)
    on all host cores, each step over a bounded sample of the stream."""
    threads = host_threads()
    sample_n = min(cfg["n_train"], 4_000_000)
    O, model, train = host_loop_model(S, cfg, args.seed, sample_n)
    lrs = O.lr_schedule(cfg["hyper"]["learning_rate"], cfg["hyper"]["decay"], args.steps + args.warmup + 1)
    lam = cfg["hyper"]["lam"]
    for e in range(args.warmup):
        model.epoch(train, float(lrs[e]), lam, threads)
    t0 = time.perf_counter()
    for e in range(args.steps):
        model.epoch(train, float(lrs[args.warmup + e]), lam, threads)
    dt = time.perf_counter() - t0
    value = sample_n * args.steps / dt
    rule = "binary16 rows and arithmetic (MASCOT, no group promoted)" if cfg["version"] == 1 else "fp32 SGD"
    line = {
        "impl": "reference", "metric": "rating updates/sec (k=128)", "value": value, "unit": "updates/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16+f32", "data": "synthetic",
        "config": {"workload": args.workload_desc, "sample": f"{sample_n} ratings per step"},
        "cpu_baseline": {"value": value, "unit": "updates/s", "cores": threads, "kind": "port",
                         "sample": f"first {sample_n} ratings of the workload per step, {threads} host threads, Hogwild, "
                                   f"AVX2+F16C loop of the as-built rule: {rule}"},
        "e2e": {"value": value, "unit": "updates/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_sample(S, cfg, seed, budget_s=12.0):
    """Bounded CPU-baseline leg of the default run (rank 0, N=1)."""
    threads = host_threads()
    n = 2_000_000
    O, model, train = host_loop_model(S, cfg, seed, n)
    lam, lr = cfg["hyper"]["lam"], cfg["hyper"]["learning_rate"]
    model.epoch(train, lr, lam, threads)
    t0 = time.perf_counter()
    reps = 0
    while True:
        model.epoch(train, lr, lam, threads)
        reps += 1
        if time.perf_counter() - t0 > budget_s or reps >= 200:
            break
    dt = time.perf_counter() - t0
    rule = "binary16 rows and arithmetic (MASCOT, no group promoted)" if cfg["version"] == 1 else "fp32 SGD"
    return {"value": n * reps / dt, "unit": "updates/s", "cores": threads, "kind": "port",
            "sample": f"{reps} passes over the first {n} ratings of the workload, {threads} host threads, Hogwild, "
                      f"AVX2+F16C loop of the as-built rule: {rule} (oracle/host_loop.cpp; the bit-exact oracle is ~25x slower)"}


# ---------------------------------------------------------------------------------------------
# the reference's CUDA build, measured here
# ---------------------------------------------------------------------------------------------
def reference_cuda_leg(S, M, cfg, workload, seed, scale=0.1, epochs=6):
    """Times oracle/_ref/quantized_mf (the reference's own sources compiled for sm_100) on a scaled copy
    of the workload, written as the TSV the reference reads.  Returns None when the binary is absent."""
    exe = os.path.join(ROOT, "oracle", "_ref", "quantized_mf")
    conv = os.path.join(PKG, "bin", "convert_ratings")
    if not (os.path.exists(exe) and os.path.exists(conv)):
        return None
    import tempfile
    sc = S.scaled(cfg, scale)
    train_t, test_t = S.generate_cuda(sc, seed=seed)
    tmp = tempfile.mkdtemp(prefix="mascot_ref_")
    try:
        tr_bin, te_bin = os.path.join(tmp, "train.bin"), os.path.join(tmp, "test.bin")
        tr_txt, te_txt = os.path.join(tmp, "ratings_train.tsv"), os.path.join(tmp, "ratings_test.tsv")
        M.write_binary_ratings(tr_bin, train_t.numpy().view(np.uint32).reshape(-1, 3), sc["users"], sc["items"])
        M.write_binary_ratings(te_bin, test_t.numpy().view(np.uint32).reshape(-1, 3), sc["users"], sc["items"])
        subprocess.check_call([conv, tr_bin, tr_txt, "tsv"]); subprocess.check_call([conv, te_bin, te_txt, "tsv"])
        hy = cfg["hyper"]
        wg = 2048
        cmd = [exe, "-i", tr_txt, "-y", te_txt, "-k", str(cfg["k"]), "-l", str(epochs), "-a", str(hy["learning_rate"]), "-d", str(hy["decay"]),
               "-b", str(hy["lam"]), "-wg", str(wg), "-bl", "128", "-v", str(cfg["version"]), "-ug", "50", "-ig", "50",
               "-s", str(hy.get("sample_ratio", 0.01)), "-it", str(hy.get("interval", 1)), "-e", str(hy.get("error_threshold", 0.001))]
        t0 = time.time()
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        wall = time.time() - t0
        m = re.search(r"(?:Parameters update per epoch|Execution time\(avg per epoch\))\s*:\s*([0-9.eE+]+)", p.stdout)
        n = int(train_t.shape[0])
        updates = wg * int(np.ceil(n / (wg * 128))) * 128
        if p.returncode != 0 or not m:
            return {"measured": False, "why": f"rc {p.returncode}: {p.stderr[-200:]}"}
        us = float(m.group(1))
        return {"measured": True, "updates_per_s": updates / (us * 1e-6), "kernel_us_per_epoch": us, "wg": wg, "epochs": epochs,
                "workload": f"{workload} scaled by {scale}: {sc['users']}x{sc['items']}, {n} ratings (ug=ig=50)", "wall_s": wall}
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)


# ---------------------------------------------------------------------------------------------
# shared pieces of both GPU arms
# ---------------------------------------------------------------------------------------------
def phase_report(n_train, steps):
    """steps: list of (total_ms, kernel_ms, check flag, groups promoted in that epoch).  Splits the window
    at the first promotion: before it every row is binary16, after it some groups are fp32."""
    out, promoted_so_far = {}, False
    phases = {"fp16": [], "promoted": []}
    for total, kern, chk, prom in steps:
        phases["promoted" if promoted_so_far else "fp16"].append((total, kern, chk))
        if prom:
            promoted_so_far = True
    for name, rows in phases.items():
        if not rows:
            continue
        plain = [k for _, k, c in rows if not c]
        check = [k for _, k, c in rows if c]
        out[name] = {"epochs": len(rows), "updates_per_s": n_train * len(rows) / (sum(t for t, _, _ in rows) * 1e-3),
                     "plain_kernel_ms": statistics.median(plain) if plain else None,
                     "check_kernel_ms": statistics.median(check) if check else None}
    return out


def time_to_rmse(rmse, cum_ms, targets):
    out = {}
    for t in targets:
        hit = next((j for j, v in enumerate(rmse) if v <= t), None)
        out[f"{t:.6g}"] = None if hit is None else {"epoch": hit + 1, "ms": round(cum_ms[hit], 2)}
    return out


def rmse_targets(workload):
    ref = REFERENCE_CUDA_BUILD_EARLIER_RUNS.get(workload)
    base = {"c4": [0.65, 0.62, 0.61], "c5": [1.40, 1.36, 1.34]}.get(workload, [])
    return base + ([ref["final_rmse"]] if ref else [])


def run_single(args, S, M, cfg, local_rank):
    import torch
    train_t, test_t = S.generate_cuda(cfg, seed=args.seed, device=f"cuda:{local_rank}")
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    n_train, n_test = train_t.shape[0], test_t.shape[0]
    extra = {"num_workers": args.workers} if args.workers else {}
    ecfg = engine_config(M, cfg, device=local_rank, seed=args.seed, **extra)
    eng = M.Engine(ecfg)
    t_setup = time.perf_counter()
    eng.set_ratings_raw(train_t.data_ptr(), n_train, test_t.data_ptr(), n_test, cfg["users"], cfg["items"])
    setup_ms = (time.perf_counter() - t_setup) * 1e3
    eng.init_factors()

    sampler = ClockSampler(local_rank)
    epoch = 0
    for _ in range(args.warmup):
        eng.train_epoch(epoch)
        epoch += 1
    rmse_before = eng.eval_rmse()

    # ---- timed region 1: stream resident in HBM ----
    sampler.start()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    dev_ms = kern_ms = 0.0
    launches = 0
    alg_bytes = 0
    steps = []
    st = None
    for _ in range(args.steps):
        st = eng.train_epoch(epoch)
        epoch += 1
        dev_ms += st.total_ms
        kern_ms += st.kernel_ms
        launches += st.kernel_launches
        alg_bytes += st.algorithmic_bytes
        steps.append((st.total_ms, st.kernel_ms, int(st.error_check), int(st.promoted_user_groups + st.promoted_item_groups)))
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    rmse_after = eng.eval_rmse()
    value = n_train * args.steps / (dev_ms * 1e-3)
    phases = phase_report(n_train, steps)

    # ---- timed region 2: end to end from host buffers ----
    e2e = None
    if not args.no_e2e:
        eng.train_epoch_streamed_raw(epoch, train_t.data_ptr(), n_train); epoch += 1      # untimed: allocates the staging buffers
        eng.eval_rmse()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        e2e_steps = max(2, min(args.steps, 5))
        for _ in range(e2e_steps):
            # H2D of this step's inputs (pinned host memory), overlapped piece by piece with the updates
            eng.train_epoch_streamed_raw(epoch, train_t.data_ptr(), n_train); epoch += 1
            eng.eval_rmse()                                         # D2H of the step's result
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t1
        e2e = {"value": n_train * e2e_steps / e2e_s, "unit": "updates/s", "h2d_bytes_per_step": int(12 * n_train),
               "d2h_bytes_per_step": int(4 * ((n_test + 511) // 512)), "steps": e2e_steps,
               "ms_per_step": 1e3 * e2e_s / e2e_steps}
    sampler.stop_flag.set()
    sampler.join(timeout=3)
    workers = int(st.workers) if st else 0
    eng.close()

    # ---- time to a target RMSE: a fresh run of the configured number of epochs, test RMSE after each ----
    convergence = None
    if not args.no_convergence:
        eng2 = M.Engine(ecfg)
        eng2.set_ratings_raw(train_t.data_ptr(), n_train, test_t.data_ptr(), n_test, cfg["users"], cfg["items"])
        eng2.init_factors()
        rm, cum, acc = [], [], 0.0
        for e in range(int(cfg["hyper"]["epoch"])):
            s2 = eng2.train_epoch(e)
            acc += s2.total_ms
            rm.append(eng2.eval_rmse()); cum.append(acc)
        eng2.close()
        convergence = {"epochs": len(rm), "final_rmse": rm[-1], "train_ms_total": acc,
                       "updates_per_s_whole_run": n_train * len(rm) / (acc * 1e-3),
                       "time_to_rmse": time_to_rmse(rm, cum, rmse_targets(args.workload)),
                       "rmse_every_5_epochs": [round(v, 5) for v in rm[4::5]]}

    # ---- roofline of the dominant kernel (the all-binary16 update kernel of a plain epoch) ----
    hbm_peak, peak_kind = measured_peak()
    fp16 = phases.get("fp16") or phases.get("promoted")
    plain_ms = fp16["plain_kernel_ms"] or (kern_ms / args.steps)
    bytes_per_update_alg = 2 * cfg["k"] * 4 if cfg["version"] in (1, 7, 8) else 2 * cfg["k"] * 8
    alg_gbs = bytes_per_update_alg * n_train / (plain_ms * 1e-3) / 1e9
    tt = traffic_table(args.workload) if args.scale == 1.0 else None
    dram_per_launch = tt["dram_bytes_per_update"] * n_train if tt and tt.get("dram_bytes_per_update") else None
    factor_bytes = (cfg["users"] + cfg["items"]) * cfg["k"] * 2
    if (tt and tt.get("l2_bytes_per_update")) or factor_bytes < 1.5 * 126e6:
        # The update kernel is bound by instruction issue and by L2 <-> SM traffic on both listed workloads (ncu: DRAM runs
        # at a quarter to four tenths of its bandwidth): its traffic is judged against a measured L2 read bandwidth
        l2_peak = max(M.probe_read_bandwidth(32 << 20, passes=60, device=local_rank) for _ in range(5))    # best of five: the clock ramps
        l2_per_update = tt["l2_bytes_per_update"] if tt and tt.get("l2_bytes_per_update") else None
        achieved = (l2_per_update * n_train / (plain_ms * 1e-3) / 1e9) if l2_per_update else alg_gbs
        roofline = {"bound": "l2", "achieved": achieved, "peak": l2_peak, "unit": "GB/s", "frac": achieved / l2_peak,
                    "traffic": dram_per_launch,
                    "peak_kind": "measured in this run: 128-bit L2-only loads over a 32 MiB L2-resident buffer (mascot_probe_read_bandwidth, best of five)",
                    "achieved_kind": ("L2<->SM bytes per update from the committed ncu capture x updates / event-timed plain-epoch kernel"
                                      if l2_per_update else "algorithmic bytes (no ncu figure for this workload)"),
                    "frac_hbm": (dram_per_launch / (plain_ms * 1e-3) / 1e9 / hbm_peak) if dram_per_launch else None,
                    "hbm_peak": hbm_peak, "hbm_peak_kind": f"of {peak_kind}",
                    "algorithmic_gbs": alg_gbs, "algorithmic_bytes_per_update": bytes_per_update_alg,
                    "warp_instructions_per_update": tt.get("warp_instructions_per_update") if tt else None,
                    "traffic_kind": ("DRAM bytes per update of the committed ncu capture x updates" +
                                     (f" (captured at scale {tt.get('scale')}: a lower bound for the full size)" if tt and tt.get("scale", 1.0) != 1.0 else "")),
                    "note": "the kernel is bound by instruction issue and L2 traffic, not by HBM (most row accesses hit L2: popular rows on "
                            "both sides); issue_slots_busy = warp instructions per update (ncu) x updates/s / (SMs x 4 schedulers x the SM "
                            "clock sampled in this run); algorithmic bytes / HBM peak is not a roofline here and is not reported as frac"}
    else:
        roofline = {"bound": "hbm", "achieved": alg_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": alg_gbs / hbm_peak,
                    "traffic": dram_per_launch, "peak_kind": f"of {peak_kind}",
                    "frac_dram_traffic": (dram_per_launch / (plain_ms * 1e-3) / 1e9 / hbm_peak) if dram_per_launch else None,
                    "algorithmic_bytes_per_update": bytes_per_update_alg,
                    "note": "achieved = algorithmic row bytes 2*k*(b_user+b_item) per update x updates / event-timed plain-epoch kernel; "
                            "factors exceed L2 on this workload"}

    ref_cuda = None
    if not args.no_reference_cuda and args.scale == 1.0:
        try:
            ref_cuda = reference_cuda_leg(S, M, cfg, args.workload, args.seed)
        except Exception as ex:      # the leg is a courtesy measurement: never lose the bench line over it
            ref_cuda = {"measured": False, "why": repr(ex)[:200]}
    if not ref_cuda or not ref_cuda.get("measured"):
        earlier = REFERENCE_CUDA_BUILD_EARLIER_RUNS.get(args.workload)
        ref_cuda = dict(ref_cuda or {}, measured=False, fallback_from_an_earlier_full_size_run=earlier)

    clocks = sampler.summary()
    if roofline.get("warp_instructions_per_update") and clocks.get("sm_mhz"):
        import torch
        sms = torch.cuda.get_device_properties(local_rank).multi_processor_count
        roofline["issue_slots_busy"] = (roofline["warp_instructions_per_update"] * n_train / (plain_ms * 1e-3)) / (sms * 4 * clocks["sm_mhz"] * 1e6)
    line = {
        "metric": "rating updates/sec (k=128)", "value": value, "unit": "updates/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16+f32", "data": "synthetic",
        "config": {"workload": args.workload_desc, "l2": "inputs larger than L2 (rating stream read once per epoch)",
                   "phases": phases, "kernel_ms_per_step": kern_ms / args.steps, "wall_ms_per_step": wall_ms / args.steps,
                   "rmse_before": rmse_before, "rmse_after": rmse_after, "workers": workers, "setup_ms": setup_ms,
                   "total_ms_kernel_ms_check_promoted_per_step": [[round(a, 2), round(b, 2), c, d] for a, b, c, d in steps],
                   "convergence": convergence, "reference_cuda_build": ref_cuda},
        "roofline": roofline,
        "clocks": clocks,
        "gpu_launches": launches,
    }
    if e2e:
        line["e2e"] = e2e
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_sample(S, cfg, args.seed)
    print(json.dumps(line), flush=True)
    return 0


def run_sharded(args, S, M, cfg, rank, world, local_rank):
    """N > 1: one process per GPU; users pinned per rank, item blocks travelling (libmascot, csrc/shard.cu)."""
    import torch
    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    # the group id of libmascot's own communicator: made by rank 0, carried by the launcher's process group
    idt = torch.zeros(M.COMM_ID_BYTES, dtype=torch.uint8, device=dev)
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(M.comm_unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, src=0)
    comm_id = bytes(idt.cpu().numpy().tobytes())
    train_t, test_t = S.generate_cuda(cfg, seed=args.seed, device=f"cuda:{local_rank}")     # same seed: same data on every rank
    torch.cuda.synchronize(); torch.cuda.empty_cache()
    n_train, n_test = int(train_t.shape[0]), int(test_t.shape[0])
    extra = {"num_workers": args.workers} if args.workers else {}
    ecfg = engine_config(M, cfg, device=local_rank, seed=args.seed, **extra)
    eng = M.Engine(ecfg)
    eng.shard_init(comm_id, rank, world, args.blocks_per_gpu, timeout_ms=120000)
    t_setup = time.perf_counter()
    eng.shard_set_ratings_raw(train_t.data_ptr(), n_train, test_t.data_ptr(), n_test, cfg["users"], cfg["items"])
    setup_ms = (time.perf_counter() - t_setup) * 1e3
    eng.init_factors()                                 # same seed: identical factors on every rank
    n_local = eng.n_train
    # this rank's own ratings as a pinned host array, for the end-to-end leg (positions in the whole array)
    local_host = None
    if not args.no_e2e:
        order = torch.from_numpy(eng.stream_order().astype(np.int64))
        local_host = torch.empty(n_local, 3, dtype=torch.int32).pin_memory()
        torch.index_select(train_t, 0, order, out=local_host)
    epoch = 0
    for _ in range(args.warmup):
        eng.shard_train_epoch(epoch); epoch += 1
    rmse_before = eng.shard_eval_rmse()
    sampler = ClockSampler(list(range(world)))      # rank 0 watches every GPU of the job
    if rank == 0:
        sampler.start()
    dist.barrier(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps, launches, st = [], 0, None
    for _ in range(args.steps):
        st = eng.shard_train_epoch(epoch); epoch += 1
        launches += st.kernel_launches
        steps.append((st.total_ms, st.kernel_ms, int(st.error_check), int(st.promoted_user_groups + st.promoted_item_groups)))
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    mine_ms = sum(s[0] for s in steps)              # CUDA events on the engine's stream, per epoch
    t = torch.tensor([mine_ms, float(launches)], dtype=torch.float64, device=dev)
    mx = t.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = t.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    total_ms, all_launches = float(mx[0].item()), int(sm[1].item())
    loc = torch.tensor([float(n_local)], dtype=torch.float64, device=dev); dist.all_reduce(loc, op=dist.ReduceOp.MAX)
    rmse_after = eng.shard_eval_rmse()
    sent = eng.shard_info()["bytes_sent"]

    # ---- end to end: every step each rank uploads its own ratings from pinned host memory again, trains
    # the epoch (all steps and hand-overs) and reads the global test RMSE back ----
    e2e = None
    if not args.no_e2e:
        eng.reload_train_raw(local_host.data_ptr(), n_local)
        eng.shard_train_epoch(epoch); epoch += 1
        eng.shard_eval_rmse()
        e2e_steps = max(2, min(args.steps, 5))
        dist.barrier(); torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(e2e_steps):
            eng.reload_train_raw(local_host.data_ptr(), n_local)          # H2D of this step's inputs
            eng.shard_train_epoch(epoch); epoch += 1
            eng.shard_eval_rmse()                                          # D2H of the step's result
        torch.cuda.synchronize()
        te = torch.tensor([time.perf_counter() - t1], dtype=torch.float64, device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s = float(te.item())
        e2e = {"value": n_train * e2e_steps / e2e_s, "unit": "updates/s", "h2d_bytes_per_step": int(12 * n_train),
               "d2h_bytes_per_step": int(16 * world + 4 * ((n_test + 511) // 512)), "steps": e2e_steps, "ms_per_step": 1e3 * e2e_s / e2e_steps,
               "timing": "wall clock between barriers, max over ranks (the upload is a host call)"}

    # ---- time to a target RMSE: fresh factors, the configured number of epochs, global RMSE after each ----
    convergence = None
    if not args.no_convergence:
        eng.close()
        eng = M.Engine(ecfg)
        idt2 = torch.zeros(M.COMM_ID_BYTES, dtype=torch.uint8, device=dev)
        if rank == 0:
            idt2.copy_(torch.frombuffer(bytearray(M.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt2, src=0)
        eng.shard_init(bytes(idt2.cpu().numpy().tobytes()), rank, world, args.blocks_per_gpu, timeout_ms=120000)
        eng.shard_set_ratings_raw(train_t.data_ptr(), n_train, test_t.data_ptr(), n_test, cfg["users"], cfg["items"])
        eng.init_factors()
        rm, cum, acc = [], [], 0.0
        for e in range(int(cfg["hyper"]["epoch"])):
            s2 = eng.shard_train_epoch(e)
            acc += s2.total_ms
            rm.append(eng.shard_eval_rmse()); cum.append(acc)
        tc = torch.tensor(cum, dtype=torch.float64, device=dev); dist.all_reduce(tc, op=dist.ReduceOp.MAX)
        cum = tc.cpu().tolist()
        convergence = {"epochs": len(rm), "final_rmse": rm[-1], "train_ms_total": cum[-1],
                       "updates_per_s_whole_run": n_train * len(rm) / (cum[-1] * 1e-3),
                       "time_to_rmse": time_to_rmse(rm, cum, rmse_targets(args.workload)),
                       "rmse_every_5_epochs": [round(v, 5) for v in rm[4::5]]}
    sampler.stop_flag.set()
    if rank == 0:
        sampler.join(timeout=3)
        hbm_peak, peak_kind = measured_peak()
        value = n_train * args.steps / (total_ms * 1e-3)
        bytes_per_update_alg = 2 * cfg["k"] * 4 if cfg["version"] in (1, 7, 8) else 2 * cfg["k"] * 8
        achieved = value * bytes_per_update_alg / 1e9
        factor_bytes = (cfg["users"] + cfg["items"]) * cfg["k"] * 2
        phases = phase_report(n_train, steps)
        line = {
            "metric": "rating updates/sec (k=128)", "value": value, "unit": "updates/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16+f32", "data": "synthetic",
            "config": {"workload": args.workload_desc,
                       "parallelism": f"users pinned on {world} GPUs, {world * args.blocks_per_gpu} item blocks travelling by ncclSend/ncclRecv "
                                      f"inside libmascot ({args.blocks_per_gpu} per GPU)",
                       "l2": "inputs larger than L2", "rmse_before": rmse_before, "rmse_after": rmse_after,
                       "item_blocks": "sorted item index s belongs to block s mod B; a block is one contiguous row range",
                       "max_ratings_on_one_rank": int(loc.item()), "nvlink_bytes_sent_rank0_per_step": sent / max(args.steps + args.warmup, 1),
                       "workers_per_gpu": int(st.workers) if st else 0, "setup_ms_rank0": setup_ms, "phases_rank0": phases,
                       "rank0_total_ms_kernel_ms_check_promoted_per_step": [[round(a, 3), round(b, 3), c, d] for a, b, c, d in steps],
                       "timing": "CUDA events on each engine's stream around every epoch, summed over the K steps, max over ranks",
                       "wall_ms_per_step_rank0": wall_ms / max(args.steps, 1), "convergence": convergence},
            "roofline": {"bound": "hbm" if factor_bytes >= 1.5 * 126e6 else "l2", "achieved": achieved, "peak": hbm_peak * world, "unit": "GB/s",
                         "frac": achieved / (hbm_peak * world), "traffic": None, "peak_kind": f"HBM copy bandwidth of {peak_kind} (x{world} GPUs)",
                         "note": "algorithmic row bytes of the whole job against the HBM peak of all GPUs; on workloads whose factors fit "
                                 "L2 the single-GPU line carries the L2 figures"},
            "clocks": sampler.summary(), "gpu_launches": all_launches, "e2e": e2e,
        }
        print(json.dumps(line), flush=True)
    eng.close()
    dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4")
    ap.add_argument("--scale", type=float, default=1.0,
                    help="shrink the workload; used only by the ncu capture recipes in profiles/, which need a small case")
    ap.add_argument("--seed", type=int, default=4)
    ap.add_argument("--workers", type=int, default=0, help="concurrent sequential workers (-wg); 0 = the engine's automatic choice")
    ap.add_argument("--blocks-per-gpu", type=int, default=1, choices=[1, 2],
                    help="N > 1: item blocks per GPU (2 = hand-overs hidden under the update kernels)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-convergence", action="store_true", help="skip the time-to-RMSE run")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip timing the reference's own CUDA build")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    S = _load("mascot_synth", os.path.join(PKG, "synth.py"))
    cfg = S.CONFIGS[args.workload]
    if args.scale != 1.0:
        cfg = S.scaled(cfg, args.scale)
    hy = cfg["hyper"]
    args.workload_desc = (f"{args.workload}: -v {cfg['version']} k={cfg['k']}, {cfg['users']}x{cfg['items']}, {cfg['n_train']} train ratings"
                          + (f", ug=ig={hy.get('user_group_num')} s={hy.get('sample_ratio')} it={hy.get('interval')} e={hy.get('error_threshold')}"
                             if cfg["version"] == 1 else ""))

    if args.impl == "reference":
        if rank == 0:
            run_reference(args, S, cfg)
        return 0

    import torch
    M = _load("mascot_binding", os.path.join(PKG, "mascot.py"))
    M.load()   # fails loudly when the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libmascot has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        return run_sharded(args, S, M, cfg, rank, world, local_rank)
    return run_single(args, S, M, cfg, local_rank)


if __name__ == "__main__":
    sys.exit(main())
