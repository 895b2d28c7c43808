#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul hot path on B200.

Workload (``config.workload``): the Q4_K decode GEMV of the reference's batch-sweep configuration --
weight [N=14336, K=4096] drawn N(0, 0.02), quantized to Q4_K; activations f32 [M, 4096] drawn N(0, 1),
quantized to Q8_K on the device.  One *step* is one pass of the hot path (``QMatMul::forward`` =
activation quantizer + GEMV) over a pool of 16 distinct weight matrices (528 MB, larger than 2x the
126 MB L2, so every launch streams its weights from HBM).  The headline value is the weight GB/s at
M = 1: canonical packed weight bytes read per second, whole job.

Printed JSON line: see the keys below; ``roofline`` is the GEMV kernel alone (CUDA events around a graph
of GEMV launches, same pool), ``e2e`` goes through the public Python API with host buffers, and
``cpu_baseline`` times the CPU oracle (a restatement of the reference's CPU QMatMul) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
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


def physical_cores() -> int:
    try:
        import psutil

        return psutil.cpu_count(logical=False) or os.cpu_count() or 1
    except Exception:
        return os.cpu_count() or 1


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def synth_weights_f32(seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((N, K)).astype(np.float32) * np.float32(0.02)


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
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
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

def cpu_reference_rate(seconds_budget: float = 12.0, copies: int = 8):
    """Times the CPU oracle's QMatMul (AVX2 arm order, all physical cores) on the same [14336,4096] Q4_K
    GEMV at M = 1, rotating over `copies` distinct weight buffers so the host LLC cannot hold them."""
    from oracle import oracle as O

    O.build()
    cores = physical_cores()
    w = synth_weights_f32(2)
    wq = O.quantize(O.Q4_K, w, nthreads=cores)
    del w
    pool = [wq.copy() for _ in range(copies)]
    x = np.random.default_rng(3).standard_normal((1, K)).astype(np.float32)
    order = O.best_order()
    for i in range(2):
        O.matmul(O.Q4_K, x, pool[i], N, order=order, nthreads=cores)
    t0 = time.perf_counter()
    launches = 0
    while True:
        for wb in pool:
            O.matmul(O.Q4_K, x, wb, N, order=order, nthreads=cores)
            launches += 1
        if time.perf_counter() - t0 > seconds_budget or launches >= 4000:
            break
    dt = time.perf_counter() - t0
    gbps = launches * WEIGHT_BYTES / dt / 1e9
    kind = "port"
    sample = (f"{launches} GEMVs (M=1) of the full [14336,4096] Q4_K matrix over {copies} distinct copies, "
              f"{dt:.1f} s, {'AVX2+FMA' if order == O.ORDER_AVX2 else 'portable'} vec_dot")
    return gbps, cores, kind, sample, dt / launches * 1e3


def run_reference(args):
    """`--impl reference`: the reference's CPU QMatMul for this path.  The Rust reference cannot be built here
    (no rustc/cargo), so this times its C restatement in oracle/ on all physical host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, args.warmup
    per_step_budget = 1.5
    from oracle import oracle as O

    O.build()
    cores = physical_cores()
    wq = O.quantize(O.Q4_K, synth_weights_f32(2), nthreads=cores)
    pool = [wq.copy() for _ in range(8)]
    x = np.random.default_rng(3).standard_normal((1, K)).astype(np.float32)
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
        "scaling": "weak", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": {"workload": "C2 Q4_K decode GEMV [14336x4096], M=1", "pool": 8, "l2": "inputs larger than LLC"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------

def run_gpu(args):
    import torch
    import torch.distributed as dist

    import lloom_b200 as lb
    from lloom_b200 import quantized as Q

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
        dist.init_process_group("nccl", device_id=dev)

    steps, warmup = args.steps, max(args.warmup, 3)
    dtype = lb.GgmlDType.Q4K
    # weights are resident and read-only from here on: let consecutive GEMV launches overlap
    __import__("lloom_b200._lib", fromlist=["lib"]).lib().lloom_b200_set_launch_overlap(1)
    # Two seeded matrices (the C2 and C4 weights), quantized by the library's host quantizer and laid
    # out as 16 distinct device buffers: distinct memory is what defeats L2, values repeat.
    base = [Q.quantize_weights_host(synth_weights_f32(seed), dtype) for seed in (2, 6)]
    pool = [lb.QTensor.from_data(base[i % 2], dtype, (N, K), dev) for i in range(POOL)]
    mats = [lb.QMatMul.from_qtensor(q) for q in pool]
    xs_host = {m: torch.from_numpy(np.random.default_rng(3).standard_normal((m, K)).astype(np.float32)).pin_memory()
               for m in SWEEP_M}
    xs = {m: xs_host[m].to(dev) for m in SWEEP_M}
    stream = torch.cuda.Stream(device=dev)

    def fwd_pass(m, outs):
        for i, mm in enumerate(mats):
            mm.qtensor.storage.fwd((N, K), xs[m], out=outs[i])

    def gemv_pass(m, act, outs):
        L = __import__("lloom_b200._lib", fromlist=["lib"]).lib()
        for i, q in enumerate(pool):
            rc = L.lloom_b200_gemv(int(dtype), q.device_ptr(), act.data_ptr(), outs[i].data_ptr(), m, N, K, N,
                                   stream.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"gemv status {rc}")

    def capture(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()  # warm (sets kernel attributes, sizes the workspace) before capture
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                fn()
        return g

    def time_graph(g, iters, warm):
        with torch.cuda.stream(stream):
            for _ in range(warm):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            if multi:
                dist.barrier()
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(iters):
                g.replay()
            e1.record(stream)
            stream.synchronize()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if multi:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    results = {}
    outs = {m: [torch.empty(m, N, dtype=torch.float32, device=dev) for _ in range(POOL)] for m in SWEEP_M}
    graphs = {}
    with torch.cuda.stream(stream):
        for m in SWEEP_M:
            graphs[m] = capture(lambda m=m: fwd_pass(m, outs[m]))

    sampler = ClockSampler(local_rank)  # runs across every device-timed leg below (headline, sweep, roofline, prefill)
    sampler.start()
    ms_total = time_graph(graphs[1], steps, warmup)
    ms_per_step = ms_total / steps
    value = world * POOL * WEIGHT_BYTES / (ms_per_step * 1e-3) / 1e9

    sweep = {}
    for m in SWEEP_M[1:]:
        it = max(steps // 2, 3)
        ms = time_graph(graphs[m], it, 3) / it
        sweep[f"M={m}"] = round(world * POOL * WEIGHT_BYTES / (ms * 1e-3) / 1e9, 1)

    # roofline leg: the GEMV kernel alone over the same pool
    with torch.cuda.stream(stream):
        act = Q.quantize_act(dtype, xs[1])
        g_gemv = capture(lambda: gemv_pass(1, act, outs[1]))
    it = max(steps, 10)
    ms_gemv = time_graph(g_gemv, it, 3) / it / POOL  # average launch duration
    peak, peak_kind = measured_peaks()
    achieved = WEIGHT_BYTES / (ms_gemv * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "traffic": GEMV_DRAM_TRAFFIC_BYTES, "peak_kind": f"of {peak_kind}",
                "kernel": "gemv_kernel<FmtQ4K, M=1, RW=1, CW=8, PIECES=false, EPI=0>", "algorithmic_bytes_per_launch": WEIGHT_BYTES,
                "us_per_launch": round(ms_gemv * 1e3, 3)}

    # prefill leg (the metric's second half): whole QMatMul::forward at M = 512 and 2048 on the C4 matrix
    # (activation quantizer + operand preparation + tcgen05 GEMM), CUDA events, output and operands larger than L2
    gemm = {}
    bf16_peak = 1627.9
    try:
        bf16_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    for m in (512, 2048):
        xg = torch.from_numpy(np.random.default_rng(7).standard_normal((m, K)).astype(np.float32)).to(dev)
        yg = torch.empty(m, N, dtype=torch.float32, device=dev)
        with torch.cuda.stream(stream):
            for _ in range(3):
                pool[1].storage.fwd((N, K), xg, out=yg)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            reps = 10
            e0.record(stream)
            for i in range(reps):
                pool[(2 * i + 1) % POOL].storage.fwd((N, K), xg, out=yg)
            e1.record(stream)
            stream.synchronize()
        ms = e0.elapsed_time(e1) / reps
        tf = 2.0 * m * N * K / (ms * 1e-3) / 1e12
        gemm[f"M={m}"] = {"us": round(ms * 1e3, 1), "tflops": round(tf, 1), "frac_of_bf16_burst": round(tf / bf16_peak, 3)}
        del xg, yg
    clocks = sampler.stop()

    # e2e leg: public API, host buffers in, host buffers out, every step
    y_host = torch.empty(POOL, 1, N, dtype=torch.float32).pin_memory()
    y_dev = torch.empty(POOL, 1, N, dtype=torch.float32, device=dev)
    x_dev = torch.empty(1, K, dtype=torch.float32, device=dev)

    # One step = pinned host activations -> device, 16 forwards through the public API, 16 outputs -> pinned host.
    # The step is captured once in a CUDA graph (copies included) and replayed, the way a decode loop would run
    # it: launched call by call from Python the step measures the interpreter (about 12 us per forward), not
    # the library.
    def e2e_body():
        x_dev.copy_(xs_host[1], non_blocking=True)
        for i, mm in enumerate(mats):
            mm.qtensor.storage.fwd((N, K), x_dev, out=y_dev[i])
        y_host.copy_(y_dev, non_blocking=True)

    g_e2e = capture(e2e_body)

    def e2e_step():
        with torch.cuda.stream(stream):
            g_e2e.replay()
        stream.synchronize()

    for _ in range(3):
        e2e_step()
    e2e_steps = max(steps, 5)
    if multi:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if multi:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * POOL * WEIGHT_BYTES / (e2e_ms * 1e-3) / 1e9
    status = Q.device_status()

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8", "data": "synthetic",
        "config": {"workload": "C2 Q4_K decode GEMV [14336x4096], M=1: one QMatMul::forward (activation quantizer fused "
                               "into the GEMV launch) per matrix", "pool": POOL, "launch_overlap": True,
                   "pool_bytes": POOL * WEIGHT_BYTES, "l2": "inputs larger than L2 (16 distinct weight buffers, 528 MB)",
                   "timing": "CUDA events around CUDA-graph replays on the launching stream",
                   "multi_gpu": "independent matrices per rank, no collective" if multi else "single GPU"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": 4 * K,
                "d2h_bytes_per_step": 4 * POOL * N, "ms_per_step": round(e2e_ms, 4),
                "how": "pinned H2D + 16 QCudaStorage.fwd + pinned D2H, captured in one CUDA graph, host-timed per replay"},
        "gpu_launches": steps * POOL,  # one fused quantize+GEMV launch per matrix
        "roofline": roofline,
        "sweep_GBps": sweep,
        "prefill_gemm_q4k": gemm,
        "device_status": status,
    }
    if rank == 0:
        if not args.no_cpu and not multi:
            v, cores, kind, sample, ms = cpu_reference_rate()
            line["cpu_baseline"] = {"value": round(v, 2), "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample,
                                    "ms_per_gemv": round(ms, 3)}
        print(json.dumps(line), flush=True)
    if multi:
        dist.barrier()
        dist.destroy_process_group()


def run_lm_head(args):
    """`--workload lm_head`: the Q6_K lm_head [128256, 4096] at M = 1, output rows sharded over the ranks and the
    logits all-gathered with NCCL (strong scaling: the matrix is fixed, each rank streams 1/G of it)."""
    import torch
    import torch.distributed as dist

    import lloom_b200 as lb
    from lloom_b200 import _lib
    from lloom_b200 import quantized as Q
    from lloom_b200.sharded import ShardPlan, gather_rows

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    n_total, k, dtype = 128256, 4096, lb.GgmlDType.Q6K
    row_bytes = k // 256 * 210
    plan = ShardPlan(n_total, world)
    lo, hi = plan.range_of(rank)
    rows = hi - lo
    chunks = []
    c0 = lo
    while c0 < hi:  # rows are drawn per 4096-row chunk so that any sharding sees the same matrix
        c1 = min(hi, (c0 // 4096 + 1) * 4096)
        blk = np.random.default_rng([4, c0 // 4096]).standard_normal((4096, k)).astype(np.float32) * np.float32(0.02)
        chunks.append(Q.quantize_weights_host(blk[c0 % 4096: c0 % 4096 + (c1 - c0)], dtype))
        c0 = c1
    shard = np.concatenate(chunks)
    copies = max(1, -(-int(2.2 * 126e6) // (rows * row_bytes)))
    pool = [lb.QTensor.from_data(shard, dtype, (rows, k), dev) for _ in range(copies)]
    _lib.lib().lloom_b200_set_launch_overlap(1)
    x = torch.from_numpy(np.random.default_rng(5).standard_normal((1, k)).astype(np.float32)).to(dev)
    steps, warmup = args.steps, max(args.warmup, 3)

    from lloom_b200.sharded import ShardedQMatMul

    def step_nccl():
        out = None
        for q in pool:
            y_local = q.fwd(x)
            out = gather_rows(y_local, plan) if world > 1 else y_local
        return out

    def time_steps(step):
        """CUDA-event time of `steps` calls of `step`, which is captured once in a CUDA graph where capture works
        (launched call by call from Python a 40 us forward is bound by the interpreter); returns (ms, how)."""
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        how, run = "eager launches", step
        side = torch.cuda.Stream(device=dev)
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    step()
            torch.cuda.synchronize()

            def run():
                g.replay()
            how = "CUDA graph replays"
            run()
        except Exception:
            torch.cuda.synchronize()
            how, run = "eager launches", step
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        t_ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([t_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t.item())
        return t_ms, how

    ms_nccl, how_nccl = time_steps(step_nccl)
    ms, gather, fused_us, how = ms_nccl, ("NCCL all-gather" if world > 1 else "none (one GPU)"), None, how_nccl
    if world > 1:
        # the same forwards with the gather fused into the GEMV (peer stores + one barrier kernel per forward)
        fused = [ShardedQMatMul(None, plan, None, local=lb.QMatMul.from_qtensor(q)) for q in pool]
        if all(f.enable_fused_gather(1) for f in fused):
            def step_fused():
                out = None
                for f in fused:
                    out = f.forward(x)
                return out

            ms_fused, how_fused = time_steps(step_fused)
            fused_us = ms_fused / steps / copies * 1e3
            if Q.device_status() != 0:
                raise RuntimeError("device status after the fused gather")
            if ms_fused < ms_nccl:
                ms, gather, how = ms_fused, "fused into the GEMV (peer stores over NVLink + barrier kernel)", how_fused
            torch.cuda.synchronize()
            dist.barrier()
            for f in fused:
                f.close()
    per_matmul_us = ms / steps / copies * 1e3
    value = n_total * row_bytes / (per_matmul_us * 1e-6) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": "q6k_lm_head_gemv_weight_GBps", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
            "config": {"workload": "C3 Q6_K lm_head GEMV [128256x4096], M=1, rows sharded over ranks, logits gathered on every rank",
                       "gather": gather, "us_per_sharded_matmul_nccl": round(ms_nccl / steps / copies * 1e3, 2),
                       "us_per_sharded_matmul_fused": None if fused_us is None else round(fused_us, 2),
                       "copies_per_rank": copies, "us_per_sharded_matmul": round(per_matmul_us, 2),
                       "per_gpu_GBps": round(value / world, 1), "timing": "CUDA events, " + how,
                       "timing_nccl": how_nccl},
            "gpu_launches": steps * copies}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_stack(args):
    """`--workload stack`: the synthetic Llama-8B-shaped decode matmul stack (C5): 32 layers of q/o [4096,4096],
    k/v [1024,4096], gate/up [14336,4096], down [4096,14336] in Q4_K plus a Q6_K lm_head [128256,4096]; a chain of
    225 independent forwards on fixed inputs of the right K (no attention / norms), M = 1 and M = 8.  FFN and lm_head
    rows are sharded over the ranks (all-gather of their outputs); q/k/v/o are replicated.  One matrix per shape is
    quantized on the host and copied into distinct device buffers per layer: distinct memory is what the step
    streams, the values repeat."""
    import torch
    import torch.distributed as dist

    import lloom_b200 as lb
    from lloom_b200 import _lib
    from lloom_b200 import quantized as Q
    from lloom_b200.sharded import ShardPlan, gather_rows

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    layers = args.layers
    H, FF, KV, V = 4096, 14336, 1024, 128256
    q4, q6 = lb.GgmlDType.Q4K, lb.GgmlDType.Q6K

    def host_matrix(seed, n, k, dtype, lo, hi):
        out = []
        c0 = lo
        while c0 < hi:
            c1 = min(hi, (c0 // 4096 + 1) * 4096)
            blk = np.random.default_rng([seed, c0 // 4096]).standard_normal((4096, k)).astype(np.float32) * np.float32(0.02)
            out.append(Q.quantize_weights_host(blk[c0 % 4096: c0 % 4096 + (c1 - c0)], dtype))
            c0 = c1
        return np.concatenate(out)

    def shard(n):
        plan = ShardPlan(n, world)
        lo, hi = plan.range_of(rank)
        return plan, lo, hi

    specs = [("q", H, H, False), ("k", KV, H, False), ("v", KV, H, False), ("o", H, H, False),
             ("gate", FF, H, True), ("up", FF, H, True), ("down", H, FF, True)]
    protos = {}
    for i, (name, n, k, sharded) in enumerate(specs):
        plan, lo, hi = shard(n) if sharded else (None, 0, n)
        protos[name] = (host_matrix(1000 + i, n, k, q4, lo, hi), hi - lo, k, plan)
    plan_v, lo, hi = shard(V)
    lm_host = host_matrix(9000, V, H, q6, lo, hi)
    weights = []  # (QTensor, plan or None)
    bytes_local = 0
    for _ in range(layers):
        for name, _, _, _ in specs:
            host, rows, k, plan = protos[name]
            weights.append((lb.QTensor.from_data(host, q4, (rows, k), dev), plan, k))
            bytes_local += host.size
    weights.append((lb.QTensor.from_data(lm_host, q6, (hi - lo, H), dev), plan_v if world > 1 else None, H))
    bytes_local += lm_host.size
    _lib.lib().lloom_b200_set_launch_overlap(1)
    steps, warmup = args.steps, max(args.warmup, 3)
    results = {}
    for m in (1, 8):
        xs = {k: torch.from_numpy(np.random.default_rng(9001).standard_normal((m, k)).astype(np.float32)).to(dev)
              for k in (H, FF)}
        outs = [torch.empty(m, w.shape[0], dtype=torch.float32, device=dev) for w, _, _ in weights]

        def step():
            for (w, plan, k), y in zip(weights, outs):
                w.storage.fwd(w.shape, xs[k], out=y)
                if plan is not None and world > 1:
                    gather_rows(y, plan)

        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            step()
            stream.synchronize()
            use_graph = world == 1
            if use_graph:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    step()
                run = g.replay
            else:
                run = step
            for _ in range(warmup):
                run()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                run()
            e1.record(stream)
            stream.synchronize()
        ms = e0.elapsed_time(e1) / steps
        tot = torch.tensor([ms, float(bytes_local)], device=dev, dtype=torch.float64)
        if world > 1:
            t_ms = tot[:1].clone()
            dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
            t_b = tot[1:].clone()
            dist.all_reduce(t_b, op=dist.ReduceOp.SUM)
            ms, total_bytes = float(t_ms.item()), float(t_b.item())
        else:
            total_bytes = float(bytes_local)
        results[m] = (ms, total_bytes)
    if rank == 0:
        ms1, tb = results[1]
        peak, kind = measured_peaks()
        print(json.dumps({
            "metric": "llama8b_decode_stack_weight_GBps", "value": round(tb / (ms1 * 1e-3) / 1e9, 1), "unit": "GB/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms1, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
            "config": {"workload": f"C5 decode matmul stack, {layers} layers + lm_head, M=1; FFN/lm_head row-sharded",
                       "launches_per_step": len(weights), "bytes_read_per_step_all_gpus": int(tb),
                       "per_gpu_frac_of_hbm": round(tb / world / (ms1 * 1e-3) / 1e9 / peak, 3), "peak_kind": f"of {kind}",
                       "M=8": {"ms_per_step": round(results[8][0], 4),
                               "GBps": round(results[8][1] / (results[8][0] * 1e-3) / 1e9, 1)},
                       "timing": "CUDA events; one CUDA graph per step" if world == 1 else "CUDA events; eager launches + NCCL all-gathers"},
            "gpu_launches": steps * len(weights)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one M=1 GEMV launch on the full [14336,4096] matrix,
# from the ncu capture summarised in profiles/gemv_q4k_m1.md.
GEMV_DRAM_TRAFFIC_BYTES = 33089280


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--workload", default="c2", choices=["c2", "lm_head", "stack"],
                    help="c2: the headline Q4_K decode GEMV; lm_head: the row-sharded Q6_K lm_head with all-gather; "
                         "stack: the 32-layer Llama-8B-shaped decode matmul stack")
    ap.add_argument("--layers", type=int, default=32, help="layers of the stack workload")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "lm_head":
        run_lm_head(args)
    elif args.workload == "stack":
        run_stack(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
