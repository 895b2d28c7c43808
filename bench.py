#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul hot path on B200.

Headline workload (``config.workload``): the Q4_K decode GEMV of the reference's batch-sweep configuration --
weight [N=14336, K=4096] drawn N(0, 0.02), quantized to Q4_K; activations f32 [M, 4096] drawn N(0, 1),
quantized to Q8_K on the device.  One *step* is one pass of the hot path (``QMatMul::forward`` =
activation quantizer + GEMV, one launch) over a pool of 16 distinct weight matrices (528 MB, larger than 2x the
126 MB L2, so every launch streams its weights from HBM).  The headline value is the weight GB/s at
M = 1: canonical packed weight bytes read per second, whole job.

One GPU: the line also carries every other configuration (``configs``: Q8_0 GEMV, the M sweep, the grouped
gate|up / q|k|v launches, the Q6_K lm_head, the prefill GEMMs of the three formats, the 32-layer decode stack)
and a ``parity`` block computed in the same run, outside the timed regions, against the CPU oracle on a row
sample of each configuration.  N > 1 GPUs (``torchrun``): every matrix of the same pool is row-sharded over
the ranks and the outputs are assembled on every rank by the gather fused into the GEMV (strong scaling), with the
NCCL all-gather figure, the sharded lm_head and the sharded stack beside it.

``roofline`` is the GEMV kernel alone (CUDA events around a graph of GEMV launches, same pool), ``e2e`` goes
through the public API with host buffers, ``cpu_baseline`` times the CPU oracle (a restatement of the
reference's CPU QMatMul) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N, K = 14336, 4096
POOL = 16
Q4K_ROW_BYTES = K // 256 * 144
WEIGHT_BYTES = N * Q4K_ROW_BYTES  # 33,030,144: algorithmic bytes of one GEMV launch
SWEEP_M = (1, 2, 4, 8)
METRIC = "q4k_decode_gemv_weight_GBps"
Q8_0, Q4_K, Q6_K = 8, 12, 14
REPEATS = 10  # event-timed regions per figure; medians are reported


def physical_cores() -> int:
    try:
        import psutil

        n = psutil.cpu_count(logical=False)
        if n:
            return n
    except Exception:
        pass
    # no psutil: count distinct (package, core) pairs; hyper-threads share one
    try:
        cores = set()
        for cpu in os.listdir("/sys/devices/system/cpu"):
            if re.fullmatch(r"cpu\d+", cpu):
                base = f"/sys/devices/system/cpu/{cpu}/topology/"
                cores.add((open(base + "physical_package_id").read().strip(), open(base + "core_id").read().strip()))
        if cores:
            return len(cores)
    except Exception:
        pass
    return os.cpu_count() or 1


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def profiled_dram_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one M = 1 GEMV launch, from the tracked ncu summary of the
    kernel instance this file times (line `dram_bytes_per_launch: <n>`); None when the summary is absent."""
    try:
        text = open(os.path.join(ROOT, "profiles", "gemv_q4k_m1.md")).read()
        m = re.search(r"dram_bytes_per_launch:\s*([0-9]+)", text)
        return int(m.group(1)) if m else None
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            time.sleep(0.3)  # the first sample takes a moment
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(smax))
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# --------------------------------------------------------------------------------------------------
# CPU legs (the only places this file touches oracle/)
# --------------------------------------------------------------------------------------------------

CPU_THREADING_NOTE = ("the oracle's restatement of utils::BarrierPool (per-worker go / done slots, spin 10,000 then park, "
                      "flat tree as the reference builds off macOS, the caller takes the last share); "
                      "threads = physical cores, as default_num_threads does")


def cpu_reference_rate(seconds_budget: float = 12.0, copies: int = 8):
    """Times the CPU oracle's QMatMul (AVX2 arm order, all physical cores) on the same [14336,4096] Q4_K
    GEMV at M = 1, rotating over `copies` distinct weight buffers so the host LLC cannot hold them."""
    from lloom_b200 import synthetic as S
    from oracle import oracle as O

    O.build()
    cores = physical_cores()
    wq = S.quantized_matrix(2, N, K, Q4_K)
    pool = [wq.copy() for _ in range(copies)]
    x = S.activations(3, 1, K)
    order = O.best_order()
    for i in range(2):
        O.matmul(O.Q4_K, x, pool[i], N, order=order, nthreads=cores)
    t0 = time.perf_counter()
    launches = 0
    while True:
        for wb in pool:
            O.matmul(O.Q4_K, x, wb, N, order=order, nthreads=cores)
            launches += 1
        if time.perf_counter() - t0 > seconds_budget:
            break
    dt = time.perf_counter() - t0
    gbps = launches * WEIGHT_BYTES / dt / 1e9
    sample = (f"{launches} GEMVs (M=1) of the full [14336,4096] Q4_K matrix over {copies} distinct copies, "
              f"{dt:.1f} s, {'AVX2+FMA' if order == O.ORDER_AVX2 else 'portable'} vec_dot")
    return gbps, cores, "port", sample, dt / launches * 1e3


def run_reference(args):
    """`--impl reference`: the reference's CPU QMatMul for this path.  The Rust reference cannot be built here
    (no rustc/cargo), so this times its C restatement in oracle/ on all physical host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, args.warmup
    per_step_budget = 1.5
    from lloom_b200 import synthetic as S
    from oracle import oracle as O

    O.build()
    cores = physical_cores()
    wq = S.quantized_matrix(2, N, K, Q4_K)
    pool = [wq.copy() for _ in range(8)]
    x = S.activations(3, 1, K)
    order = O.best_order()

    def step():
        # a bounded sample of the workload's step: one GEMV on each of 8 of the 16 pool matrices
        for wb in pool:
            O.matmul(O.Q4_K, x, wb, N, order=order, nthreads=cores)
        return len(pool)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    launches = 0
    for _ in range(steps):
        launches += step()
        if time.perf_counter() - t0 > per_step_budget * steps + 60:
            break
    dt = time.perf_counter() - t0
    value = launches * WEIGHT_BYTES / dt / 1e9
    sample = f"{launches} GEMVs (M=1) over 8 distinct copies of the [14336,4096] Q4_K matrix per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt / max(steps, 1) * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": {"workload": "C2 Q4_K decode GEMV [14336x4096], M=1", "pool": 8, "l2": "inputs larger than LLC"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                         "threading": CPU_THREADING_NOTE},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# Parity figures (oracle = the checker; never inside a timed region)
# --------------------------------------------------------------------------------------------------

def parity_figures(O, dt, x, wq_rows, got, act_got=None):
    """Oracle comparison of `got` [m, rows] = x @ W[rows]^T: the figures the specification asks for, none asserted
    here except by the caller.  A = sum of magnitudes of the f32 summands the reference's AVX2 arm adds."""
    cores = physical_cores()
    rows = wq_rows.shape[0]
    ref = O.matmul(dt, x, wq_rows, rows, nthreads=cores).astype(np.float64)
    A = O.matmul_absum(dt, x, wq_rows, rows, nthreads=cores).astype(np.float64)
    got = np.asarray(got, np.float64)
    err = np.abs(got - ref)
    rms = np.sqrt(np.mean(ref * ref, axis=1, keepdims=True))
    out = {
        "outputs": int(ref.size),
        "max_err_over_A": float((err / np.maximum(A, 1e-30)).max()),
        "max_err_over_max_ref_1e-3rms": float((err / np.maximum(np.abs(ref), 1e-3 * rms)).max()),
        "max_rel": float((err / np.maximum(np.abs(ref), 1e-30)).max()),
        "max_abs": float(err.max()),
        "share_cancelling": float(np.mean(np.abs(ref) < A / 32)),
    }
    solid = np.abs(ref) >= A / 32
    out["max_rel_noncancelling"] = float((err[solid] / np.abs(ref[solid])).max()) if solid.any() else 0.0
    if act_got is not None:
        out["act_blocks_byte_equal"] = bool(np.array_equal(act_got, O.quantize_act(dt, x)))
    out["ok"] = bool(out["max_err_over_A"] <= 1e-6 and out["max_rel_noncancelling"] <= 1e-5
                     and out.get("act_blocks_byte_equal", True))
    return out


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------

class Timer:
    """CUDA-event timing on the launching stream; graphs for launch-bound regions."""

    def __init__(self, torch, dist, stream, dev, multi):
        self.torch, self.dist, self.stream, self.dev, self.multi = torch, dist, stream, dev, multi
        self.graphs = []

    def capture(self, fn):
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.stream):
            fn()  # warm (sets kernel attributes, sizes the workspace) before capture
            self.stream.synchronize()
            with torch.cuda.graph(g, stream=self.stream):
                fn()
        self.graphs.append(g)
        return g.replay

    def release(self):
        """Destroys every captured graph.  A graph that holds a captured NCCL collective keeps a reference on the
        communicator, and tearing the process group down while such a graph is alive never returns."""
        self.torch.cuda.synchronize()
        for g in self.graphs:
            g.reset()
        self.graphs = []
        self.torch.cuda.synchronize()

    def region(self, run, iters):
        """One timed region of `iters` calls: barrier + synchronize on both sides, max over ranks; ms."""
        torch = self.torch
        with torch.cuda.stream(self.stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.stream.synchronize()
            if self.multi:
                self.dist.barrier()
            torch.cuda.synchronize()
            e0.record(self.stream)
            for _ in range(iters):
                run()
            e1.record(self.stream)
            self.stream.synchronize()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if self.multi:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def median(self, run, iters, warm=3, repeats=REPEATS):
        """Median / min / max over `repeats` timed regions of `iters` calls each; ms per call."""
        with self.torch.cuda.stream(self.stream):
            for _ in range(warm):
                run()
        ts = [self.region(run, iters) / iters for _ in range(repeats)]
        return float(np.median(ts)), float(min(ts)), float(max(ts))


def stat(ms_tuple, per=1.0):
    med, lo, hi = ms_tuple
    return {"us": round(med * 1e3 / per, 3), "us_min": round(lo * 1e3 / per, 3), "us_max": round(hi * 1e3 / per, 3)}


def run_gpu(args):
    import torch
    import torch.distributed as dist

    import lloom_b200 as lb
    from lloom_b200 import _lib
    from lloom_b200 import quantized as Q
    from lloom_b200 import synthetic as S

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    multi = world > 1
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if multi:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keeps NCCL's version banner off stdout, where the result line goes
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    # weights are resident and read-only from here on: let consecutive GEMV launches overlap
    L.lloom_b200_set_launch_overlap(1)
    stream = torch.cuda.Stream(device=dev)
    T = Timer(torch, dist, stream, dev, multi)
    steps, warmup = args.steps, max(args.warmup, 3)
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    if multi:
        return run_sharded(args, torch, dist, lb, Q, S, L, T, rank, world, dev, stream, hbm_peak, peak_kind)

    dtype = lb.GgmlDType.Q4K
    # Two seeded matrices (the C2 and C4 weights), quantized by the library's host quantizer and laid
    # out as 16 distinct device buffers: distinct memory is what defeats L2, values repeat.
    base = [S.quantized_matrix(seed, N, K, Q4_K) for seed in (2, 6)]
    pool = [lb.QTensor.from_data(base[i % 2], dtype, (N, K), dev) for i in range(POOL)]
    mats = [lb.QMatMul.from_qtensor(q) for q in pool]
    xs_np = {m: S.activations(3, m, K) for m in SWEEP_M}
    xs_host = {m: torch.from_numpy(xs_np[m]).pin_memory() for m in SWEEP_M}
    xs = {m: xs_host[m].to(dev) for m in SWEEP_M}
    outs = {m: [torch.empty(m, N, dtype=torch.float32, device=dev) for _ in range(POOL)] for m in SWEEP_M}

    def fwd_pass(m):
        for i, mm in enumerate(mats):
            mm.qtensor.storage.fwd((N, K), xs[m], out=outs[m][i])

    def group_pass(m, g):
        for i in range(0, POOL, g):
            Q.forward_group(mats[i:i + g], xs[m], outs=outs[m][i:i + g])

    graphs = {m: T.capture(lambda m=m: fwd_pass(m)) for m in SWEEP_M}

    sampler = ClockSampler(local_rank)  # runs across every device-timed leg below
    sampler.start()
    # ---- headline: exactly `steps` steps after `warmup` warm-up steps, one timed region ----
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            graphs[1]()
    ms_total = T.region(graphs[1], steps)
    ms_per_step = ms_total / steps
    value = POOL * WEIGHT_BYTES / (ms_per_step * 1e-3) / 1e9
    rep = T.median(graphs[1], steps, warm=0)
    repeat_stats = {"regions": REPEATS, "steps_per_region": steps, "ms_per_step_median": round(rep[0], 5),
                    "ms_per_step_min": round(rep[1], 5), "ms_per_step_max": round(rep[2], 5)}

    configs = {}
    # ---- C2 sweep and grouped launches ----
    it = max(steps // 2, 5)
    c2 = {}
    for m in SWEEP_M:
        t = T.median(graphs[m], it)
        c2[f"M={m}"] = dict(stat(t, POOL), GBps=round(WEIGHT_BYTES / (t[0] * 1e-3 / POOL) / 1e9, 1),
                            frac_hbm=round(WEIGHT_BYTES / (t[0] * 1e-3 / POOL) / 1e9 / hbm_peak, 4))
    for g, name in ((2, "pair (gate|up)"), (4, "quad")):
        for m in (1, 8):
            run = T.capture(lambda m=m, g=g: group_pass(m, g))
            t = T.median(run, it)
            c2[f"M={m} grouped {name}"] = dict(stat(t, POOL), GBps=round(WEIGHT_BYTES / (t[0] * 1e-3 / POOL) / 1e9, 1),
                                               frac_hbm=round(WEIGHT_BYTES / (t[0] * 1e-3 / POOL) / 1e9 / hbm_peak, 4),
                                               note="per matrix; the matrices of a group share one activation read")
    configs["C2_q4k_gemv_14336x4096"] = c2
    sweep = {k: v["GBps"] for k, v in c2.items() if k in ("M=2", "M=4", "M=8")}

    # ---- roofline leg: the GEMV kernel alone over the same pool ----
    with torch.cuda.stream(stream):
        act = Q.quantize_act(dtype, xs[1])

    def gemv_pass():
        for i, q in enumerate(pool):
            rc = L.lloom_b200_gemv(int(dtype), q.device_ptr(), act.data_ptr(), outs[1][i].data_ptr(), 1, N, K, N,
                                   stream.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"gemv status {rc}")

    t = T.median(T.capture(gemv_pass), max(steps, 10))
    us_launch = t[0] * 1e3 / POOL
    achieved = WEIGHT_BYTES / (us_launch * 1e-6) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                "frac": round(achieved / hbm_peak, 4), "traffic": profiled_dram_traffic(), "peak_kind": f"of {peak_kind}",
                "kernel": "gemv_kernel<FmtQ4K, M=1, RW=1, CW=8, PIECES=false, EPI=0, GROUP=false> (single matrix per launch)",
                "algorithmic_bytes_per_launch": WEIGHT_BYTES, "us_per_launch": round(us_launch, 3),
                "us_per_launch_min_max": [round(t[1] * 1e3 / POOL, 3), round(t[2] * 1e3 / POOL, 3)],
                "grouped_frac": {"pair": c2["M=1 grouped pair (gate|up)"]["frac_hbm"], "quad": c2["M=1 grouped quad"]["frac_hbm"]}}

    parity = {}
    from oracle import oracle as O  # the checker, used between timed regions only

    O.build()
    rng = np.random.default_rng(12345)
    # parity of C2 (all four batch sizes, 1024-row sample of pool matrix 0)
    sample = np.sort(rng.choice(N, 1024, replace=False))
    wsub = np.ascontiguousarray(base[0][sample])
    torch.cuda.synchronize()
    for m in SWEEP_M:
        aq = Q.quantize_act(dtype, xs[m]).cpu().numpy()
        parity[f"C2 M={m}"] = parity_figures(O, Q4_K, xs_np[m], wsub, outs[m][0].cpu().numpy()[:, sample], aq)

    # ---- C1: Q8_0 [8192, 2048], M = 1 ----
    n1, k1 = 8192, 2048
    w1 = S.quantized_matrix(0, n1, k1, Q8_0)
    pool1 = [lb.QTensor.from_data(w1, Q8_0, (n1, k1), dev) for _ in range(POOL)]
    x1_np = S.activations(1, 1, k1)
    x1 = torch.from_numpy(x1_np).to(dev)
    y1 = [torch.empty(1, n1, dtype=torch.float32, device=dev) for _ in range(POOL)]

    def c1_pass():
        for i, q in enumerate(pool1):
            q.storage.fwd((n1, k1), x1, out=y1[i])

    t = T.median(T.capture(c1_pass), max(steps, 10))
    b1 = w1.size
    configs["C1_q8_0_gemv_8192x2048"] = {"M=1": dict(stat(t, POOL), GBps=round(b1 / (t[0] * 1e-3 / POOL) / 1e9, 1),
                                                    frac_hbm=round(b1 / (t[0] * 1e-3 / POOL) / 1e9 / hbm_peak, 4),
                                                    algorithmic_bytes=int(b1))}
    torch.cuda.synchronize()
    parity["C1 M=1"] = parity_figures(O, Q8_0, x1_np, w1, y1[0].cpu().numpy(), Q.quantize_act(lb.GgmlDType.Q8_0, x1).cpu().numpy())
    # Q8_0 prefill GEMM on the same matrix (tcgen05, per-32 drains)
    gemm_cfg = {}

    def gemm_leg(qts, dt, n, k, ms, seed, key, check_m=None):
        res = {}
        for m in ms:
            xg_np = S.activations(seed, m, k)
            xg = torch.from_numpy(xg_np).to(dev)
            yg = torch.empty(m, n, dtype=torch.float32, device=dev)
            idx = [0]

            def call():
                idx[0] = (idx[0] + 1) % len(qts)
                qts[idx[0]].storage.fwd((n, k), xg, out=yg)

            t = T.median(call, 6, warm=3)
            tf = 2.0 * m * n * k / (t[0] * 1e-3) / 1e12
            entry = dict(stat(t), tflops=round(tf, 1), frac_bf16_burst=round(tf / bf16_peak, 4))
            for q in qts:
                q.storage.build_prefill_image((n, k))
            t = T.median(call, 6, warm=3)
            tf = 2.0 * m * n * k / (t[0] * 1e-3) / 1e12
            entry["prebuilt_image"] = dict(stat(t), tflops=round(tf, 1), frac_bf16_burst=round(tf / bf16_peak, 4))
            for q in qts:
                q.storage.drop_prefill_image()
            res[f"M={m}"] = entry
            if check_m is not None and m in check_m:
                call()
                torch.cuda.synchronize()
                rr = np.sort(rng.choice(m, min(m, 16), replace=False))
                cc = np.sort(rng.choice(n, min(n, 1536), replace=False))
                host = qts[idx[0]].data_host
                parity[f"{key} M={m}"] = parity_figures(O, dt, xg_np[rr], np.ascontiguousarray(host[cc]),
                                                        yg.cpu().numpy()[np.ix_(rr, cc)])
            del xg, yg
        return res

    for q in pool1:
        q.data_host = w1
    configs["J1_q8_0_gemm_8192x2048"] = gemm_leg(pool1[:4], Q8_0, n1, k1, (64, 512, 2048), 7, "J1 Q8_0 GEMM", check_m=(64, 512))
    del pool1, y1

    # ---- C4: Q4_K prefill GEMM [14336, 4096], M = 512 and 2048 (pool matrices built from seed 6) ----
    c4_pool = [pool[i] for i in (1, 3, 5, 7)]
    for q in c4_pool:
        q.data_host = base[1]
    configs["C4_q4k_gemm_14336x4096"] = gemm_leg(c4_pool, Q4_K, N, K, (512, 2048), 7, "C4", check_m=(512, 2048))

    # ---- C3: Q6_K lm_head [128256, 4096], M = 1, one GPU ----
    n3 = 128256
    w3 = S.quantized_matrix(4, n3, K, Q6_K)
    q3 = lb.QTensor.from_data(w3, Q6_K, (n3, K), dev)
    x3_np = S.activations(5, 1, K)
    x3 = torch.from_numpy(x3_np).to(dev)
    y3 = torch.empty(1, n3, dtype=torch.float32, device=dev)

    def c3_pass():
        for _ in range(4):
            q3.storage.fwd((n3, K), x3, out=y3)

    t = T.median(T.capture(c3_pass), 5)
    b3 = w3.size
    configs["C3_q6k_lm_head_128256x4096"] = {"M=1": dict(stat(t, 4), GBps=round(b3 / (t[0] * 1e-3 / 4) / 1e9, 1),
                                                        frac_hbm=round(b3 / (t[0] * 1e-3 / 4) / 1e9 / hbm_peak, 4),
                                                        algorithmic_bytes=int(b3), l2="one matrix of 431 MB > L2")}
    torch.cuda.synchronize()
    s3 = np.sort(rng.choice(n3, 4096, replace=False))
    parity["C3 M=1"] = parity_figures(O, Q6_K, x3_np, np.ascontiguousarray(w3[s3]), y3.cpu().numpy()[:, s3],
                                      Q.quantize_act(lb.GgmlDType.Q6K, x3).cpu().numpy())
    # Q6_K prefill GEMM on a 14336-row slice of it
    q6_pool = [lb.QTensor.from_data(w3[i * N:(i + 1) * N], Q6_K, (N, K), dev) for i in range(4)]
    for i, q in enumerate(q6_pool):
        q.data_host = w3[i * N:(i + 1) * N]
    configs["J1_q6k_gemm_14336x4096"] = gemm_leg(q6_pool, Q6_K, N, K, (64, 512, 2048), 7, "J1 Q6_K GEMM", check_m=(64, 512))
    del q6_pool
    # the three added formats on the same two frames (Q5_K: Q4_K's kernel; Q4_0 / Q5_0: Q8_0's), M = 512 and 2048
    for dt, name, n_, k_ in ((13, "q5k", N, K), (2, "q4_0", n1, k1), (6, "q5_0", n1, k1)):
        wx = S.quantized_matrix(20 + dt, n_, k_, dt)
        qx = [lb.QTensor.from_data(wx, dt, (n_, k_), dev) for _ in range(2)]
        for q in qx:
            q.data_host = wx
        configs[f"J1_{name}_gemm_{n_}x{k_}"] = gemm_leg(qx, dt, n_, k_, (512, 2048), 7, f"J1 {name} GEMM", check_m=(512,))
        del qx, wx

    # ---- C5: decode matmul stack (32 layers + lm_head), M = 1 and 8, one CUDA graph per step ----
    configs["C5_decode_stack"] = stack_leg(args, torch, lb, Q, S, T, O, dev, hbm_peak, parity, rng, lm_head=(q3, w3))
    clocks = sampler.stop()

    # ---- e2e legs: public API, host buffers in, host buffers out, every step ----
    y_host = torch.empty(POOL, 1, N, dtype=torch.float32).pin_memory()
    y_dev = torch.empty(POOL, 1, N, dtype=torch.float32, device=dev)
    x_dev = torch.empty(1, K, dtype=torch.float32, device=dev)

    # (a) One step = pinned host activations -> device, 16 forwards through the public API, 16 outputs -> pinned host,
    # captured once in a CUDA graph (copies included) and replayed, the way a decode loop would run it: the outputs go
    # back four at a time on a second stream while the next forwards run (every byte still leaves inside the step).
    copy_stream = torch.cuda.Stream(device=dev)

    def e2e_body():
        x_dev.copy_(xs_host[1], non_blocking=True)
        for i, mm in enumerate(mats):
            mm.qtensor.storage.fwd((N, K), x_dev, out=y_dev[i])
            if i % 4 == 3:
                done = torch.cuda.Event()
                done.record(stream)
                copy_stream.wait_event(done)
                with torch.cuda.stream(copy_stream):
                    y_host[i - 3:i + 1].copy_(y_dev[i - 3:i + 1], non_blocking=True)
        joined = torch.cuda.Event()
        joined.record(copy_stream)
        stream.wait_event(joined)

    g_e2e = T.capture(e2e_body)

    def host_timed(step_fn, n_steps):
        for _ in range(3):
            step_fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n_steps):
            step_fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / n_steps

    def e2e_graph_step():
        with torch.cuda.stream(stream):
            g_e2e()
        stream.synchronize()

    e2e_ms = host_timed(e2e_graph_step, max(steps, 5))
    e2e_value = POOL * WEIGHT_BYTES / (e2e_ms * 1e-3) / 1e9

    # (b) call by call through the C++ host layer (QMatMul::forward of qcuda_storage.cpp: its own workspace, the
    # legacy default stream), no graph: what a host that launches every forward itself sees
    import ctypes as C

    handles = []
    for i in range(POOL):
        h = C.c_void_p()
        rc = L.lloom_b200_host_qtensor_from_data(local_rank, None, base[i % 2].ctypes.data, base[i % 2].size, int(dtype), N, K,
                                                 C.byref(h))
        if rc != 0:
            raise RuntimeError(L.lloom_b200_host_last_error().decode())
        handles.append(h)

    def e2e_percall_step():  # everything on the legacy default stream, which is also the host layer's
        x_dev.copy_(xs_host[1])  # host -> device
        for i, h in enumerate(handles):
            rc = L.lloom_b200_host_qmatmul_forward(h, x_dev.data_ptr(), 1, y_dev[i].data_ptr())
            if rc != 0:
                raise RuntimeError(L.lloom_b200_host_last_error().decode())
        y_host.copy_(y_dev)  # device -> host, synchronous

    torch.cuda.synchronize()
    percall_ms = host_timed(e2e_percall_step, max(steps, 5))
    torch.cuda.synchronize()
    percall_equal = bool(np.array_equal(y_host[0].numpy(), outs[1][0].cpu().numpy()))
    for h in handles:
        L.lloom_b200_host_qtensor_free(h)
    status = Q.device_status()

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8", "data": "synthetic",
        "config": {"workload": "C2 Q4_K decode GEMV [14336x4096], M=1: one QMatMul::forward (activation quantizer fused "
                               "into the GEMV launch) per matrix", "pool": POOL, "launch_overlap": True,
                   "pool_bytes": POOL * WEIGHT_BYTES, "l2": "inputs larger than L2 (16 distinct weight buffers, 528 MB)",
                   "timing": f"CUDA events around CUDA-graph replays on the launching stream; other figures: median of "
                             f"{REPEATS} timed regions",
                   "multi_gpu": "single GPU"},
        "clocks": clocks,
        "repeat_stats": repeat_stats,
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": 4 * K,
                "d2h_bytes_per_step": 4 * POOL * N, "ms_per_step": round(e2e_ms, 4),
                "how": "pinned H2D + 16 QCudaStorage.fwd + pinned D2H (four outputs at a time on a second stream, joined "
                       "before the step ends), captured in one CUDA graph, host-timed per replay",
                "per_call_cpp_host_layer": {"value": round(POOL * WEIGHT_BYTES / (percall_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                                            "ms_per_step": round(percall_ms, 4), "same_bits_as_python_api": percall_equal,
                                            "how": "H2D copy + 16 QMatMul::forward of the C++ host layer, launched "
                                                   "call by call (no graph) + synchronous D2H copy, host-timed"}},
        "gpu_launches": steps * POOL,  # one fused quantize+GEMV launch per matrix
        "roofline": roofline,
        "sweep_GBps": sweep,
        "prefill_gemm_q4k": {k: {"us": v["us"], "tflops": v["tflops"], "frac_of_bf16_burst": v["frac_bf16_burst"],
                                 "prebuilt_image": v["prebuilt_image"]}
                             for k, v in configs["C4_q4k_gemm_14336x4096"].items()},
        "configs": configs,
        "parity": {"all_ok": all(v["ok"] for v in parity.values()), "bounds": {"max_err_over_A": 1e-6, "max_rel_noncancelling": 1e-5},
                   "cases": parity},
        "device_status": status,
    }
    if not args.no_cpu:
        v, cores, kind, sample, ms = cpu_reference_rate()
        line["cpu_baseline"] = {"value": round(v, 2), "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample,
                                "ms_per_gemv": round(ms, 3), "threading": CPU_THREADING_NOTE}
    print(json.dumps(line), flush=True)


STACK_SPECS = [("q", 4096, 4096, False), ("k", 1024, 4096, False), ("v", 1024, 4096, False), ("o", 4096, 4096, False),
               ("gate", 14336, 4096, True), ("up", 14336, 4096, True), ("down", 4096, 14336, True)]


def stack_leg(args, torch, lb, Q, S, T, O, dev, hbm_peak, parity, rng, lm_head):
    """The synthetic Llama-8B-shaped decode matmul stack on one GPU: 32 layers of q/o [4096,4096], k/v [1024,4096],
    gate/up [14336,4096], down [4096,14336] in Q4_K plus the Q6_K lm_head [128256,4096]; 225 forwards on fixed inputs
    of the right K (no attention / norms), one CUDA graph per step.  One matrix per shape is quantized on the host
    (seed 1000 + index) and copied into a distinct device buffer per layer: distinct memory is what the step streams,
    the values repeat.  Also timed with q|k|v and gate|up behind grouped launches."""
    layers = args.layers
    protos = {name: S.quantized_matrix(1000 + i, n, k, Q4_K) for i, (name, n, k, _) in enumerate(STACK_SPECS)}
    layer_w = []
    total_bytes = 0
    for _ in range(layers):
        d = {}
        for name, n, k, _ in STACK_SPECS:
            d[name] = lb.QMatMul.from_qtensor(lb.QTensor.from_data(protos[name], Q4_K, (n, k), dev))
            total_bytes += protos[name].size
        layer_w.append(d)
    q3, w3 = lm_head
    lm = lb.QMatMul.from_qtensor(q3)
    total_bytes += w3.size
    out = {"layers": layers, "matmuls_per_step": 7 * layers + 1, "bytes_per_step": int(total_bytes)}
    for m in (1, 8):
        x_np = {k: S.activations(9001, m, k) for k in (4096, 14336)}
        xs = {k: torch.from_numpy(v).to(dev) for k, v in x_np.items()}
        ys = [{name: torch.empty(m, n, dtype=torch.float32, device=dev) for name, n, _, _ in STACK_SPECS} for _ in range(layers)]
        y_lm = torch.empty(m, 128256, dtype=torch.float32, device=dev)

        def step_single():
            for d, y in zip(layer_w, ys):
                for name, n, k, _ in STACK_SPECS:
                    d[name].qtensor.storage.fwd((n, k), xs[k], out=y[name])
            lm.qtensor.storage.fwd((128256, 4096), xs[4096], out=y_lm)

        def step_grouped():
            for d, y in zip(layer_w, ys):
                Q.forward_group([d["q"], d["k"], d["v"]], xs[4096], outs=[y["q"], y["k"], y["v"]])
                d["o"].qtensor.storage.fwd((4096, 4096), xs[4096], out=y["o"])
                Q.forward_group([d["gate"], d["up"]], xs[4096], outs=[y["gate"], y["up"]])
                d["down"].qtensor.storage.fwd((4096, 14336), xs[14336], out=y["down"])
            lm.qtensor.storage.fwd((128256, 4096), xs[4096], out=y_lm)

        res = {}
        for label, fn in (("one_launch_per_matmul", step_single), ("qkv_and_gate_up_grouped", step_grouped)):
            t = T.median(T.capture(fn), 3)
            res[label] = {"ms_per_step": round(t[0], 4), "ms_min": round(t[1], 4), "ms_max": round(t[2], 4),
                          "GBps": round(total_bytes / (t[0] * 1e-3) / 1e9, 1),
                          "frac_hbm": round(total_bytes / (t[0] * 1e-3) / 1e9 / hbm_peak, 4)}
        out[f"M={m}"] = res
        # parity of the step's own outputs (last layer + lm_head), row samples
        torch.cuda.synchronize()
        for name, n, k, _ in STACK_SPECS:
            if name in ("v", "up"):
                continue  # same shapes as k and gate
            s = np.sort(rng.choice(n, min(n, 512), replace=False))
            parity[f"C5 {name} M={m}"] = parity_figures(O, Q4_K, x_np[k], np.ascontiguousarray(protos[name][s]),
                                                        ys[-1][name].cpu().numpy()[:, s])
        s = np.sort(rng.choice(128256, 1024, replace=False))
        parity[f"C5 lm_head M={m}"] = parity_figures(O, Q6_K, x_np[4096], np.ascontiguousarray(w3[s]), y_lm.cpu().numpy()[:, s])
        del ys, y_lm
    return out


def run_sharded(args, torch, dist, lb, Q, S, L, T, rank, world, dev, stream, hbm_peak, peak_kind):
    """N > 1: strong scaling of the row-sharded path.  Headline: the 16-matrix C2 pool with every matrix split by rows
    over the ranks and each forward's outputs assembled on every rank by peer stores fused into the GEMV, completion
    flags published by the GEMV's last CTA and awaited by a one-warp kernel (the NCCL all-gather figure beside it)."""
    from lloom_b200.sharded import ShardedQMatMul, ShardPlan, forward_after_gather, gather_rows

    steps, warmup = args.steps, max(args.warmup, 3)
    # a peer that never publishes must not cost the default two seconds per wait (ranks are in step to within a few
    # milliseconds here: every leg starts behind a collective)
    Q.set_wait_limit_ns(1_000_000_000)

    def check_status(where):
        st = torch.tensor([float(Q.device_status())], device=dev)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        if int(st.item()) != 0:
            raise SystemExit(f"device status {int(st.item())} after {where}: a bounded device-side wait ran out")

    plan = ShardPlan(N, world)
    lo, hi = plan.range_of(rank)
    base = [S.quantized_rows(seed, lo, hi, K, Q4_K) for seed in (2, 6)]
    x_np = S.activations(3, 1, K)
    x = torch.from_numpy(x_np).to(dev)

    def sharded_pool(host, dt, n, k, copies):
        return [ShardedQMatMul(None, ShardPlan(n, world), None,
                               local=lb.QMatMul.from_qtensor(lb.QTensor.from_data(host, dt, (host.shape[0], k), dev)))
                for _ in range(copies)]

    pool = [sharded_pool(base[i % 2], Q4_K, N, K, 1)[0] for i in range(POOL)]
    with torch.cuda.stream(stream):
        for s in pool:
            assert s.enable_fused_gather(8)
    last = {}

    def fused_pass(m_x):  # every forward followed by its own wait kernel
        for s in pool:
            last["y"] = s.forward(m_x)

    def chained_pass(m_x):
        # the decode chain's shape: every forward waits, in its own prologue, for the gather of the forward before it
        # (as if it consumed those rows); one wait kernel closes the step
        prev = None
        for i, s in enumerate(pool):
            last["y_chain"] = s.forward(m_x, after=prev, wait=(i == len(pool) - 1))
            prev = s

    def nccl_pass(m_x):
        for s in pool:
            last["y_nccl"] = gather_rows(s._local.forward(m_x), s.plan)

    run_waitk = T.capture(lambda: fused_pass(x))
    run_fused = T.capture(lambda: chained_pass(x))
    check_status("the first sharded forwards")
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            run_fused()
    sampler = ClockSampler(dev.index)
    sampler.start()
    ms_total = T.region(run_fused, steps)
    ms_per_step = ms_total / steps
    value = POOL * WEIGHT_BYTES / (ms_per_step * 1e-3) / 1e9
    rep = T.median(run_fused, steps, warm=0)
    t_waitk = T.median(run_waitk, max(steps // 2, 5))
    try:
        run_nccl = T.capture(lambda: nccl_pass(x))
        how_nccl = "CUDA graph"
    except Exception:  # capture of the collective refused: launch it eagerly
        torch.cuda.synchronize()
        run_nccl, how_nccl = (lambda: nccl_pass(x)), "eager launches"
    t_nccl = T.median(run_nccl, max(steps // 2, 5))
    # same-run parity: the gathered rows of the last matrix equal the unsharded forward bit for bit (rank 0 holds the
    # full matrix for this check only), and both gathers agree
    torch.cuda.synchronize()
    y_f = last["y_chain"].clone()
    y_w = last["y"].clone()
    y_n = last["y_nccl"].clone()
    full_host = S.quantized_matrix((2, 6)[(POOL - 1) % 2], N, K, Q4_K)
    y_full = lb.QMatMul.from_qtensor(lb.QTensor.from_data(full_host, Q4_K, (N, K), dev)).forward(x)
    torch.cuda.synchronize()
    bits_equal = bool(torch.equal(y_f, y_full) and torch.equal(y_n, y_full) and torch.equal(y_w, y_full))
    sharded = {"C2_pool_fused_gather_consumer_waits": dict(stat(rep, POOL), GBps=round(value, 1)),
               "C2_pool_fused_gather_wait_kernel_each": dict(stat(t_waitk, POOL),
                                                             GBps=round(WEIGHT_BYTES / (t_waitk[0] * 1e-3 / POOL) / 1e9, 1)),
               "C2_pool_nccl_all_gather": dict(stat(t_nccl, POOL), GBps=round(WEIGHT_BYTES / (t_nccl[0] * 1e-3 / POOL) / 1e9, 1),
                                               timing=how_nccl)}
    for s in pool:
        s.close()
    del pool

    # ---- lm_head (C3): Q6_K [128256, 4096], M = 1 ----
    n3 = 128256
    plan3 = ShardPlan(n3, world)
    lo3, hi3 = plan3.range_of(rank)
    w3 = S.quantized_rows(4, lo3, hi3, K, Q6_K)
    copies = max(2, -(-int(2.2 * 126e6) // w3.size))
    lm_pool = sharded_pool(w3, Q6_K, n3, K, copies)
    x3 = torch.from_numpy(S.activations(5, 1, K)).to(dev)
    with torch.cuda.stream(stream):
        for s in lm_pool:
            assert s.enable_fused_gather(8)

    def lm_fused():
        for s in lm_pool:
            last["lm"] = s.forward(x3)

    def lm_nccl():
        for s in lm_pool:
            last["lm_nccl"] = gather_rows(s._local.forward(x3), s.plan)

    check_status("the C2 pool")
    t_f = T.median(T.capture(lm_fused), 5)
    try:
        run = T.capture(lm_nccl)
    except Exception:
        torch.cuda.synchronize()
        run = lm_nccl
    t_n = T.median(run, 5)
    b3 = n3 * (K // 256 * 210)
    torch.cuda.synchronize()
    lm_equal = bool(torch.equal(last["lm"], last["lm_nccl"]))
    sharded["lm_head_sharded"] = {"fused_gather": dict(stat(t_f, copies), GBps=round(b3 / (t_f[0] * 1e-3 / copies) / 1e9, 1)),
                                  "nccl_all_gather": dict(stat(t_n, copies), GBps=round(b3 / (t_n[0] * 1e-3 / copies) / 1e9, 1)),
                                  "fused_equals_nccl_bits": lm_equal, "rows_per_gpu": hi3 - lo3, "copies_per_rank": copies}
    lm_one = lm_pool[0]
    for s in lm_pool[1:]:
        s.close()

    # ---- decode stack (C5): FFN and lm_head sharded, q/k/v/o replicated; one CUDA graph per step ----
    layers = args.layers
    protos = {}
    for i, (name, n, k, is_sharded) in enumerate(STACK_SPECS):
        if is_sharded:
            a, b = ShardPlan(n, world).range_of(rank)
            protos[name] = S.quantized_rows(1000 + i, a, b, k, Q4_K)
        else:
            protos[name] = S.quantized_matrix(1000 + i, n, k, Q4_K)
    layer_w = []
    bytes_local = 0
    with torch.cuda.stream(stream):
        for _ in range(layers):
            d = {}
            for name, n, k, is_sharded in STACK_SPECS:
                mm = lb.QMatMul.from_qtensor(lb.QTensor.from_data(protos[name], Q4_K, (protos[name].shape[0], k), dev))
                if is_sharded:
                    d[name] = ShardedQMatMul(None, ShardPlan(n, world), None, local=mm)
                    assert d[name].enable_fused_gather(8)
                else:
                    d[name] = mm
                bytes_local += protos[name].size
            layer_w.append(d)
    bytes_local += w3.size
    tb = torch.tensor([float(bytes_local)], device=dev, dtype=torch.float64)
    dist.all_reduce(tb, op=dist.ReduceOp.SUM)
    total_bytes = float(tb.item())
    stack = {"layers": layers, "bytes_read_per_step_all_gpus": int(total_bytes),
             "sharded": "gate, up, down, lm_head by rows; q, k, v, o replicated"}
    for m in (1, 8):
        xs = {k: torch.from_numpy(S.activations(9001, m, k)).to(dev) for k in (4096, 14336)}
        ys = [{name: torch.empty(m, n, dtype=torch.float32, device=dev) for name, n, _, s in STACK_SPECS if not s}
              for _ in range(layers)]

        def step():
            prev = None  # the sharded matmul whose gather the next forward waits for in its own prologue
            for d, y in zip(layer_w, ys):
                for name in ("q", "k", "v", "o"):
                    n, k = d[name].qtensor.shape
                    if prev is not None and m <= 2:
                        forward_after_gather(d[name], xs[k], prev, out=y[name])
                        prev = None
                    else:
                        d[name].qtensor.storage.fwd((n, k), xs[k], out=y[name])
                chain = m <= 2
                d["gate"].forward(xs[4096], wait=not chain)
                d["up"].forward(xs[4096], after=d["gate"] if chain else None, wait=not chain)
                d["down"].forward(xs[14336], after=d["up"] if chain else None, wait=not chain)
                prev = d["down"] if chain else None
            last["stack_lm"] = lm_one.forward(xs[4096], after=prev if m <= 2 else None, wait=True)

        run_step = T.capture(step)
        check_status(f"the first stack steps, M={m}")
        t = T.median(run_step, 3)
        stack[f"M={m}"] = {"ms_per_step": round(t[0], 4), "ms_min": round(t[1], 4), "ms_max": round(t[2], 4),
                           "aggregate_GBps": round(total_bytes / (t[0] * 1e-3) / 1e9, 1),
                           "per_gpu_frac_hbm": round(total_bytes / world / (t[0] * 1e-3) / 1e9 / hbm_peak, 4),
                           "sync": "each consumer waits for its producer's gather in its own prologue" if m <= 2
                                   else "one wait kernel per sharded matmul"}
        del ys
    sharded["stack_sharded"] = stack
    clocks = sampler.stop()
    status = Q.device_status()
    st = torch.tensor([float(status)], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    for d in layer_w:
        for name in ("gate", "up", "down"):
            d[name].close()
    lm_one.close()

    # e2e at N GPUs: host activations in, gathered outputs of the 16 sharded forwards back to the host, per step
    # (the pool is gone: rebuild a small one for this leg)
    pool = [sharded_pool(base[i % 2], Q4_K, N, K, 1)[0] for i in range(POOL)]
    with torch.cuda.stream(stream):
        for s in pool:
            assert s.enable_fused_gather(1)
    x_host = torch.from_numpy(x_np).pin_memory()
    x_dev = torch.empty(1, K, dtype=torch.float32, device=dev)
    y_dev = torch.empty(POOL, 1, N, dtype=torch.float32, device=dev)
    y_host = torch.empty(POOL, 1, N, dtype=torch.float32).pin_memory()

    def e2e_body():
        x_dev.copy_(x_host, non_blocking=True)
        for i, s in enumerate(pool):
            y_dev[i].copy_(s.forward(x_dev))
        y_host.copy_(y_dev, non_blocking=True)

    g = T.capture(e2e_body)

    def e2e_step():
        with torch.cuda.stream(stream):
            g()
        stream.synchronize()

    for _ in range(3):
        e2e_step()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_e2e = max(steps, 5)
    for _ in range(n_e2e):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / n_e2e
    tt = torch.tensor([e2e_ms], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    e2e_ms = float(tt.item())
    for s in pool:
        s.close()

    if rank == 0:
        achieved = WEIGHT_BYTES / world / (ms_per_step * 1e-3 / POOL) / 1e9  # per GPU: its shard's bytes per forward time
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "i8", "data": "synthetic",
            "config": {"workload": "C2 Q4_K decode GEMV [14336x4096], M=1, every matrix row-sharded over the ranks, outputs "
                                   "assembled on every rank", "pool": POOL, "launch_overlap": True, "gpus_active": world,
                       "rows_per_gpu": hi - lo,
                       "multi_gpu": "all-gather of the [1, 14336] f32 outputs fused into the GEMV: peer stores over NVLink, "
                                    "completion flags published by the GEMV's last CTA; each forward waits for the "
                                    "gather before it in its own prologue, one wait kernel closes the step (a wait "
                                    "kernel per forward and the NCCL all-gather are timed beside it)",
                       "l2": "16 distinct weight buffers; at 8 GPUs a rank's 16 shards (66 MB) fit its L2 -- the price of "
                             "strong scaling on a 33 MB matrix",
                       "timing": "CUDA events around CUDA-graph replays, barrier + synchronize on both sides, max over ranks"},
            "clocks": clocks,
            "repeat_stats": {"regions": REPEATS, "steps_per_region": steps, "ms_per_step_median": round(rep[0], 5),
                             "ms_per_step_min": round(rep[1], 5), "ms_per_step_max": round(rep[2], 5)},
            "e2e": {"value": round(POOL * WEIGHT_BYTES / (e2e_ms * 1e-3) / 1e9, 1), "unit": "GB/s", "h2d_bytes_per_step": 4 * K,
                    "d2h_bytes_per_step": 4 * POOL * N, "ms_per_step": round(e2e_ms, 4),
                    "how": "per rank: pinned H2D + 16 sharded forwards (fused gather) + pinned D2H of the gathered outputs, "
                           "one CUDA graph, host-timed, max over ranks"},
            "gpu_launches": steps * (POOL + 1),  # per rank: one GEMV per forward + the step's closing wait kernel
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                         "frac": round(achieved / hbm_peak, 4), "traffic": None, "peak_kind": f"of {peak_kind}",
                         "note": "per GPU: shard bytes / time per sharded forward (the exchange included); latency-bound"},
            "sharded": sharded,
            "parity": {"all_ok": bool(bits_equal and lm_equal), "gathered_equals_unsharded_bits": bits_equal,
                       "lm_head_fused_equals_nccl_bits": lm_equal},
            "device_status": int(st.item()),
        }
        print(json.dumps(line), flush=True)
    # the result is out: nothing below may keep the job alive (a stuck teardown would otherwise run into the
    # launcher's limit); the watchdog ends the process with status 0 if the orderly path takes over a minute
    import threading

    dog = threading.Timer(60.0, lambda: os._exit(0))
    dog.daemon = True
    dog.start()
    last.clear()
    T.release()
    dist.barrier()
    dist.destroy_process_group()
    dog.cancel()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--layers", type=int, default=32, help="layers of the decode-stack leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
