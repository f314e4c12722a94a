#!/usr/bin/env python
"""Benchmark of the matmul path: fp16 GEMM TFLOP/s + int4 GEMV HBM GB/s against the B200 roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0). A "step" is one product of the named workload:
  N = 1   fp16 dense GEMM M=N=K=4096, fp32 accumulate (the workload the metric is quoted on);
          the line also carries the other single-GPU workloads under "configs" (int4 GEMV/GEMM,
          batched matmul, fp32 1024^3, bf16 16384^3) each with its own roofline figures.
  N > 1   bf16 GEMM M=N=K=16384 with B split by N-columns over the ranks; every rank computes its
          column block and stores each finished tile into the full C of every rank through
          peer-mapped memory (the all-gather is fused into the epilogue); strong scaling. The line
          carries the same product timed on one GPU in the same run, the efficiency that follows, a
          parity check of the gathered C against the CPU checker, the batch-sharded batched matmul
          and a comparator that does the same job with an NCCL all-gather.
`value` is timed with CUDA events on the launching stream with inputs resident in HBM; `e2e` is
the same product through the operator API from pinned host buffers, copies inside the timed
region. `--impl reference` times the CPU restatement of the same product on the host cores (the
reference project ships no matmul of its own to run).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
NOMINAL_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch, taken from ncu captures of these kernels in separate runs
# (a run under a profiler is never a bench value, so this cannot be measured here). None: no capture of that kernel.
NCU_TRAFFIC = {
    "gemm_f16_4096": 105.9e6,  # 89.0 MB read + 16.9 MB written
    "int4_gemv_m1": 23.3e6,    # read; nothing is written back within the kernel
    "int4_gemm_tc_m64": 23.8e6,  # read; the 1.4 MB of output stay in L2
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()  # exact PID of the sampler this object started
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        """Median clock and the throttle reasons of the samples taken between t0 and t1 (host clock)."""
        rows = []
        for ts, line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                rows.append((ts, float(parts[0]), float(parts[1]), float(parts[2]), parts[3:7]))
            except ValueError:
                continue
        inside = [r for r in rows if t0 <= r[0] <= t1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": rows[0][2] if rows else None, "reasons": [], "samples": 0,
                    "note": "no sample fell inside the timed region"}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in inside for i in range(4) if r[4][i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": max(r[2] for r in inside),
                "power_w_max": max(r[3] for r in inside), "reasons": reasons, "samples": len(inside)}


# ----------------------------------------------------------------------------- helpers
def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def time_reps(torch, dist, world, fn, steps, warmup, min_span_s, max_reps=400):
    """`warmup` untimed calls of fn(i), then `reps` regions of exactly `steps` calls each, back to back, every region
    between its own pair of CUDA events; barrier + synchronize before the first and after the last region. The number
    of regions is chosen so that the whole span lasts about `min_span_s` (so that clock samples fall inside it).
    Returns (list of ms per region, max over ranks each; host time at start; host time at end)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    # one probe region to size the run
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for i in range(steps):
        fn(warmup + i)
    p1.record()
    torch.cuda.synchronize()
    probe_ms = max(p0.elapsed_time(p1), 1e-3)
    reps = int(min(max_reps, max(1, math.ceil(min_span_s * 1e3 / probe_ms))))
    if world > 1:
        t = torch.tensor([reps], dtype=torch.int64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        reps = int(t.item())
        dist.barrier()
        torch.cuda.synchronize()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    t0 = time.time()
    k = warmup + steps
    for e0, e1 in events:
        e0.record()
        for i in range(steps):
            fn(k + i)
        e1.record()
        k += steps
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    t1 = time.time()
    ms = [e0.elapsed_time(e1) for e0, e1 in events]
    if world > 1:
        t = torch.tensor(ms, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = [float(x) for x in t.tolist()]
    return ms, t0, t1


def time_region(torch, dist, world, fn, steps, warmup):
    """`warmup` untimed and exactly `steps` timed calls of fn(i) in one region; returns ms (max over ranks)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    t1 = time.time()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, t0, t1


def time_graph(torch, fn, sets, steps, warmup):
    """Device time per launch with the host launch path taken out: `fn(i)` for one full rotation of the
    buffer sets is captured in a CUDA graph and the graph is replayed until `steps` launches have run.
    Returns microseconds per launch."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(max(warmup, 3)):
            fn(i)  # also lets the library create its per-device state outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(sets):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
        replays = max(1, (steps + sets - 1) // sets)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    return e0.elapsed_time(e1) / (replays * sets) * 1e3


def synth_f16(shape, std, seed, stream, dtype):
    """Seeded normal(0, std) in 16-bit storage; large matrices tile a 4096 x 4096 seeded block."""
    import numpy as np
    import torch
    from beantensor_b200 import synth
    r, c = shape
    br, bc = min(r, 4096), min(c, 4096)
    block = synth.normal((br, bc), std, seed, stream).astype(np.float32)
    t = torch.from_numpy(block).to(dtype)
    if (br, bc) != (r, c):
        t = t.repeat((r + br - 1) // br, (c + bc - 1) // bc)[:r, :c].contiguous()
    return t


def tensor_roofline(peaks, tflops, span_s, clocks):
    """Tensor-bound roofline entry. The denominator follows from the run: the sustained cuBLAS figure when the timed
    span was long enough for the power cap to act and a clock sample inside it shows sw_power_cap, the burst figure
    otherwise. Both fractions are printed."""
    capped = "sw_power_cap" in (clocks or {}).get("reasons", [])
    sustained = span_s >= 0.5 and capped
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    return {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
            "peak_source": f"{peaks['_source']} cuBLAS bf16 {'sustained' if sustained else 'burst'} "
                           f"(timed span {span_s:.2f} s, sw_power_cap {'seen' if capped else 'not seen'} in it)",
            "frac_of_burst_peak": tflops / peaks["bf16_tflops"], "frac_of_sustained_peak": tflops / peaks["bf16_tflops_sustained"],
            "frac_nominal": tflops / NOMINAL_TFLOPS}


def spread(ms_list, steps):
    per = sorted(m / steps for m in ms_list)
    return {"regions": len(per), "ms_per_step_median": statistics.median(per), "ms_per_step_min": per[0], "ms_per_step_max": per[-1]}


# ----------------------------------------------------------------------------- CPU arm
WORKLOAD_N1 = "fp16 dense GEMM M=N=K=4096, row-major A[M,K] B[K,N], fp32 accumulate, fp16 out"
METRIC_N1 = "fp16 GEMM TFLOP/s (M=N=K=4096)"
METRIC_MULTI = "bf16 GEMM TFLOP/s (M=N=K=16384, B sharded by N-columns, all-gather of C included)"


def workload_multi(world):
    return f"bf16 GEMM M=N=K=16384, B split by N-columns over {world} ranks, all-gather of C fused into the epilogue (stores over NVLink)"


def cpu_gemm_sample(n: int, target_seconds: float, max_rows: int = 4096):
    """Sizes a row slab of the n^3 product so that one CPU product takes about `target_seconds`.
    Returns (A, B, rows, cores); A holds max_rows rows."""
    import numpy as np
    from beantensor_b200 import synth
    from oracle import oracle as O
    O.build()
    cores = O.threads()
    blk = min(n, 4096)
    B = synth.normal((blk, blk), n ** -0.5, 1, 1).astype(np.float16).astype(np.float32)
    A = synth.normal((max_rows, blk), n ** -0.5, 1, 0).astype(np.float16).astype(np.float32)
    if blk != n:  # large matrices tile a seeded 4096 x 4096 block, as the GPU arm's inputs do
        B = np.ascontiguousarray(np.tile(B, (n // blk, n // blk)))
        A = np.ascontiguousarray(np.tile(A, (1, n // blk)))
    probe_rows = 384
    O.gemm_f32_threads(A[:probe_rows], B, cores)
    t = time.time()
    O.gemm_f32_threads(A[:probe_rows], B, cores)
    per_row = (time.time() - t) / probe_rows
    rows = int(min(max_rows, max(probe_rows, target_seconds / max(per_row, 1e-9))))
    rows -= rows % 96
    rows = max(rows, 96)
    return A, B, rows, cores


CPU_KIND_NOTE = "CPU restatement (register-blocked AVX-512 FMA kernel, rows split over host threads); the reference ships no matmul"


def run_reference_arm(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import oracle as O
    multi = args.gpus > 1
    n = 16384 if multi else 4096
    total = args.steps + args.warmup
    budget = 150.0  # seconds for the whole run
    A, B, rows, cores = cpu_gemm_sample(n, min(20.0, budget / max(total, 1)))
    for _ in range(args.warmup):
        O.gemm_f32_threads(A[:rows], B, cores)
    t0 = time.time()
    for _ in range(args.steps):
        O.gemm_f32_threads(A[:rows], B, cores)
    dt = time.time() - t0
    flops = 2.0 * rows * n * n * args.steps
    tflops = flops / dt / 1e12
    sample = f"{rows} of {n} rows of the {n}^3 product per step (16-bit inputs widened to fp32), {args.steps} steps"
    line = {
        "impl": "reference", "metric": METRIC_MULTI if multi else METRIC_N1, "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / max(args.steps, 1) * 1e3,
        "higher_is_better": True, "scaling": "strong" if multi else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_multi(args.gpus) if multi else WORKLOAD_N1, "arm": CPU_KIND_NOTE + "; host cores only, no GPU is used"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm, N = 1
def gemm_buffers(torch, dtype, n, sets):
    std = n ** -0.5
    bufs = []
    for s in range(sets):
        a = synth_f16((n, n), std, 1, 2 * s, dtype).cuda()
        b = synth_f16((n, n), std, 1, 2 * s + 1, dtype).cuda()
        c = torch.empty((n, n), dtype=dtype, device="cuda")
        bufs.append((a, b, c))
    return bufs


def bench_e2e_gemm(torch, ops, dtype, n, steps, warmup):
    """Host buffers in pinned memory -> device -> product -> host, every step.

    The three legs of a step run on three streams (upload, product, download) over two device buffer
    sets, so that the upload of step i+1 and the download of step i-1 overlap the product of step i, as a
    caller feeding a stream of products would arrange it. Every step still uploads both operands and
    downloads the whole result; the timed region covers all of it."""
    std = n ** -0.5
    ha = synth_f16((n, n), std, 1, 0, dtype).pin_memory()
    hb = synth_f16((n, n), std, 1, 1, dtype).pin_memory()
    hc = [torch.empty((n, n), dtype=dtype).pin_memory() for _ in range(2)]
    dev = [tuple(torch.empty((n, n), dtype=dtype, device="cuda") for _ in range(3)) for _ in range(2)]
    main = torch.cuda.current_stream()
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    uploaded = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    for e in downloaded + computed:
        e.record(main)

    def step(i):
        s = i & 1
        da, db, dc = dev[s]
        up.wait_event(computed[s])       # the product that last read this set's operands is done
        with torch.cuda.stream(up):
            da.copy_(ha, non_blocking=True)
            db.copy_(hb, non_blocking=True)
            uploaded[s].record(up)
        main.wait_event(uploaded[s])
        main.wait_event(downloaded[s])   # the previous result in this set has left the device
        ops.matmul_gpu(da, db, dc)
        computed[s].record(main)
        down.wait_event(computed[s])
        with torch.cuda.stream(down):
            hc[s].copy_(dc, non_blocking=True)
            downloaded[s].record(down)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    for i in range(steps):
        step(warmup + i)
    for e in downloaded:
        main.wait_event(e)  # the last downloads finish before the closing event
    e1.record(main)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), 2 * n * n * 2, n * n * 2


def bench_int4(torch, ops, peaks, M, steps, warmup):
    import numpy as np
    from beantensor_b200 import synth
    N, K, G = 11008, 4096, 128
    w_bytes = N * K // 2
    sets = max(2, (2 * L2_BYTES) // w_bytes + 1)  # rotate weight copies so every launch streams from HBM
    w = synth.pack_int4(synth.int4((N, K), 2))
    s = synth.uniform((N, K // G), 0.005, 0.02, 2, 1).astype(np.float16)
    act = synth.normal((M, K), 1.0, 2, 2).astype(np.float16)
    ws = [torch.from_numpy(w).cuda() for _ in range(sets)]
    ss = [torch.from_numpy(s).cuda() for _ in range(sets)]
    a = torch.from_numpy(act).cuda()
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")

    def step(i):
        ops.matmul_int4_gpu(a, ws[i % sets], ss[i % sets], out, G)

    ms, _, _ = time_region(torch, None, 1, step, steps, warmup)
    us_host = ms / steps * 1e3  # one Python call per launch: bounded by the host launch path
    us = time_graph(torch, step, sets, steps, warmup)
    # The same launch with one weight copy only (23 MB: it stays in the 126 MB L2), reported beside the HBM figure.
    us_l2 = time_graph(torch, lambda i: ops.matmul_int4_gpu(a, ws[0], ss[0], out, G), sets, steps, warmup)
    algo = w_bytes + N * (K // G) * 2 + M * K * 2 + M * N * 2
    gbs = algo / (us * 1e-6) / 1e9
    return {"workload": f"int4 weight-only matmul M={M} N=11008 K=4096 group=128", "us_per_launch": us,
            "us_per_launch_host_loop": us_host, "launch": f"CUDA graph of {sets} launches, replayed",
            "l2_resident": {"us_per_launch": us_l2, "gbs": algo / (us_l2 * 1e-6) / 1e9,
                            "what": "one weight copy, re-read from L2 by every launch; not the value, not in the roofline"},
            "algorithmic_bytes": algo, "value": gbs, "unit": "GB/s",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "frac_nominal": gbs / NOMINAL_HBM_GBS,
                         "traffic": NCU_TRAFFIC["int4_gemv_m1"] if M == 1 else NCU_TRAFFIC["int4_gemm_tc_m64"] if M == 64 else None,
                         "traffic_source": "ncu capture of a separate run" if M in (1, 64) else None},
            "l2": f"{sets} rotating weight copies ({sets * w_bytes >> 20} MiB > L2)"}


def bench_bmm(torch, ops, peaks, steps, warmup):
    Bn, M, N, K = 64, 512, 512, 128
    sets = 6  # 6 x 48 MiB > L2
    bufs = []
    for s in range(sets):
        a = synth_f16((Bn * M, K), K ** -0.5, 3, 2 * s, torch.float16).view(Bn, M, K).cuda()
        b = synth_f16((Bn * K, N), K ** -0.5, 3, 2 * s + 1, torch.float16).view(Bn, K, N).cuda()
        bufs.append((a, b, torch.empty((Bn, M, N), dtype=torch.float16, device="cuda")))

    def step(i):
        a, b, c = bufs[i % sets]
        ops.bmm_gpu(a, b, c)

    ms, _, _ = time_region(torch, None, 1, step, steps, warmup)
    us_host = ms / steps * 1e3
    us = time_graph(torch, step, sets, steps, warmup)
    us_l2 = time_graph(torch, lambda i: ops.bmm_gpu(*bufs[0]), sets, steps, warmup)  # one buffer set (48 MiB): stays in L2
    algo = (Bn * M * K + Bn * K * N + Bn * M * N) * 2
    gbs = algo / (us * 1e-6) / 1e9
    tf = 2.0 * Bn * M * N * K / (us * 1e-6) / 1e12
    return {"workload": "batched fp16 matmul [64,512,128]x[64,128,512]", "us_per_launch": us, "us_per_launch_host_loop": us_host,
            "launch": f"CUDA graph of {sets} launches, replayed", "algorithmic_bytes": algo,
            "l2_resident": {"us_per_launch": us_l2, "gbs": algo / (us_l2 * 1e-6) / 1e9,
                            "what": "one buffer set, re-read from and re-written into L2 by every launch; not the value, not in the roofline"},
            "value": gbs, "unit": "GB/s", "tflops": tf,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "frac_nominal": gbs / NOMINAL_HBM_GBS, "traffic": None,
                         "traffic_note": "a capture of one launch sees the reads only (16.9 MB): the 33.6 MB of C are still in "
                                         "the 126 MB L2 when the kernel ends, so no per-launch DRAM figure is quoted"},
            "l2": f"{sets} rotating buffer sets ({sets * algo >> 20} MiB > L2)"}


def bench_f32(torch, ops, peaks, steps, warmup):
    import numpy as np
    from beantensor_b200 import synth
    n = 1024
    a = torch.from_numpy(synth.uniform((n, n), -1, 1, 0, 0).astype(np.float32)).cuda()
    b = torch.from_numpy(synth.uniform((n, n), -1, 1, 0, 1).astype(np.float32)).cuda()
    c = torch.empty((n, n), dtype=torch.float32, device="cuda")
    ms, _, _ = time_region(torch, None, 1, lambda i: ops.matmul_gpu(a, b, c), steps, warmup)
    us_host = ms / steps * 1e3
    us = time_graph(torch, lambda i: ops.matmul_gpu(a, b, c), 8, steps, warmup)
    tf = 2.0 * n ** 3 / (us * 1e-6) / 1e12
    # The tensor cores do three TF32 products per fp32 product; the roofline counts the flops once (2 M N K), against
    # the bf16 burst peak as the nearest measured tensor figure (a TF32 product runs at half the bf16 rate).
    return {"workload": "fp32 dense matmul M=N=K=1024 (3xTF32 split)", "us_per_launch": us, "us_per_launch_host_loop": us_host,
            "launch": "CUDA graph of 8 products (2 kernels each: operand split, product), replayed",
            "value": tf, "unit": "TFLOP/s", "launches_per_step": 2,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
                         "peak_source": peaks["_source"] + " cuBLAS bf16 burst; flops counted once (2*M*N*K), the kernel issues 3x as "
                                        "TF32 at half the bf16 rate, so 1/6 of this peak is the ceiling of the method",
                         "l2_to_sm_bytes": 201e6, "traffic": None}}


def run_single(args, peaks):
    import torch
    from beantensor_b200 import ops
    torch.cuda.set_device(0)
    ops.init(0)
    sampler = ClockSampler(0)
    sampler.start()  # nvidia-smi needs a moment to come up: start it before the inputs are built
    n = args.size
    flops = 2.0 * n ** 3
    sets = 4 if n <= 4096 else 2  # 4 x 96 MiB of A, B, C > 126 MiB L2
    bufs = gemm_buffers(torch, torch.float16, n, sets)

    def step(i):
        a, b, c = bufs[i % sets]
        ops.matmul_gpu(a, b, c)

    ms_list, t0, t1 = time_reps(torch, None, 1, step, args.steps, args.warmup, args.min_span)
    ops.check_device_status(0)
    clocks = sampler.summary(t0, t1)
    sp = spread(ms_list, args.steps)
    ms_step = sp["ms_per_step_median"]
    tflops = flops / (ms_step * 1e-3) / 1e12
    roof = tensor_roofline(peaks, tflops, t1 - t0, clocks)
    roof["traffic"] = NCU_TRAFFIC["gemm_f16_4096"] if n == 4096 else None
    roof["traffic_source"] = "ncu capture of a separate run"
    if clocks.get("sm_mhz"):
        roof["us_x_sm_mhz"] = ms_step * 1e3 * clocks["sm_mhz"]  # launch time in SM cycles: comparable across clock states

    # The library's own figure for the same product on the same buffers, timed the same way (informational).
    def lib_step(i):
        a, b, c = bufs[i % sets]
        torch.matmul(a, b, out=c)

    lib_ms, lt0, lt1 = time_reps(torch, None, 1, lib_step, args.steps, args.warmup, args.min_span)
    lib_clocks = sampler.summary(lt0, lt1)
    lib_sp = spread(lib_ms, args.steps)
    lib_tf = flops / (lib_sp["ms_per_step_median"] * 1e-3) / 1e12
    library = {"what": "torch.matmul (cuBLAS) on the same buffers, same timing scheme; informational", "value": lib_tf, "unit": "TFLOP/s",
               "ms_per_step": lib_sp["ms_per_step_median"], "ratio_ours_over_library": tflops / lib_tf, "clocks": lib_clocks}
    del bufs
    torch.cuda.empty_cache()

    e2e_steps = max(3, min(args.steps, 20))
    e2e_ms, h2d, d2h = bench_e2e_gemm(torch, ops, torch.float16, n, e2e_steps, 3)
    e2e_tflops = flops / (e2e_ms / e2e_steps * 1e-3) / 1e12

    extra = []
    if not args.headline_only:
        sub_steps = max(20, min(args.steps, 400))
        for M in (1, 8, 64):
            extra.append(bench_int4(torch, ops, peaks, M, sub_steps, 10))
        extra.append(bench_bmm(torch, ops, peaks, sub_steps, 10))
        extra.append(bench_f32(torch, ops, peaks, sub_steps, 10))
        bb = gemm_buffers(torch, torch.bfloat16, 16384, 1)
        big_ms, bt0, bt1 = time_reps(torch, None, 1, lambda i: ops.matmul_gpu(*bb[0]), 5, 3, args.min_span, 40)
        big_clocks = sampler.summary(bt0, bt1)
        big_sp = spread(big_ms, 5)
        tfb = 2.0 * 16384 ** 3 / (big_sp["ms_per_step_median"] * 1e-3) / 1e12
        rb = tensor_roofline(peaks, tfb, bt1 - bt0, big_clocks)
        rb["traffic"] = None
        extra.append({"workload": "bf16 dense GEMM M=N=K=16384, 1 GPU", "ms_per_launch": big_sp["ms_per_step_median"], "value": tfb,
                      "unit": "TFLOP/s", "timing": big_sp, "clocks": big_clocks, "roofline": rb})
        del bb
        torch.cuda.empty_cache()
    sampler.stop()

    cpu = None
    if not args.no_cpu:
        from oracle import oracle as O
        A, B, rows, cores = cpu_gemm_sample(4096, 10.0)
        O.gemm_f32_threads(A[:rows], B, cores)
        t = time.time()
        O.gemm_f32_threads(A[:rows], B, cores)
        dt = time.time() - t
        cpu = {"value": 2.0 * rows * 4096 * 4096 / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
               "sample": f"{rows} of 4096 rows of the fp16 4096^3 product, inputs widened to fp32, one timed run of {dt:.1f} s; " + CPU_KIND_NOTE}

    line = {
        "metric": METRIC_N1 if n == 4096 else f"fp16 GEMM TFLOP/s (M=N=K={n})", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD_N1 if n == 4096 else WORKLOAD_N1.replace("4096", str(n)),
                   "l2": f"{sets} rotating A/B/C sets ({sets * 3 * n * n * 2 >> 20} MiB > 126 MiB L2)",
                   "kernel": args.force_kernel or "library choice",
                   "timing": f"{sp['regions']} regions of exactly {args.steps} steps back to back, each between its own CUDA events; "
                             "value is the median region"},
        "timing": sp,
        "roofline": roof,
        "library_same_run": library,
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        "gpu_launches": args.steps * sp["regions"],
        "clocks": clocks,
        "configs": extra,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm, N > 1
class SharedBuffer:
    """Device memory that every rank of the job can address: allocated with btm_ipc_alloc, handles exchanged
    through the process group, peers mapped with btm_ipc_open. `table` is the C array of all ranks' bases."""

    def __init__(self, L, dist, local_rank, rank, world, nbytes):
        import ctypes as C
        from beantensor_b200.errors import raise_for_status
        self.L, self.dist, self.dev, self.rank, self.world = L, dist, local_rank, rank, world
        self.ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        raise_for_status(L.btm_ipc_alloc(local_rank, nbytes, C.byref(self.ptr), handle))
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw)
        self.peers = []
        for r in range(world):
            if r == rank:
                self.peers.append(self.ptr.value)
            else:
                p = C.c_void_p()
                raise_for_status(L.btm_ipc_open(local_rank, handles[r], C.byref(p)))
                self.peers.append(p.value)
        self.table = (C.c_void_p * world)(*self.peers)

    def release(self):
        import ctypes as C
        import torch
        self.dist.barrier()
        torch.cuda.synchronize()
        for r in range(self.world):
            if r != self.rank:
                self.L.btm_ipc_close(self.dev, C.c_void_p(self.peers[r]))
        self.dist.barrier()
        self.L.btm_ipc_free(self.dev, self.ptr)


def stream_barrier(torch, dist, flag):
    """Cross-rank barrier in stream order: a one-element all-reduce. The host does not wait."""
    dist.all_reduce(flag)


def checksum(torch, c):
    """Position-weighted sum of the 16-bit words of a matrix, exact in int64; equal matrices give equal sums and a
    permutation of rows or columns changes it."""
    n_rows, n_cols = c.shape
    wc = (torch.arange(n_cols, device=c.device, dtype=torch.int64) % 1021) + 1
    total = torch.zeros((), dtype=torch.int64, device=c.device)
    for r0 in range(0, n_rows, 1024):
        blk = c[r0:r0 + 1024].view(torch.int16).to(torch.int64)
        wr = (torch.arange(r0, r0 + blk.shape[0], device=c.device, dtype=torch.int64) % 1019) + 1
        total += ((blk * wc).sum(dim=1) * wr).sum()
    return total


def bench_bmm_sharded(torch, dist, ops, rank, world, peaks, steps, weak):
    """cfg4 sharded by batch index, no collective: every rank multiplies its own batch slice. `weak`: 64 products per
    rank instead of 64 in all. Parity of every rank's slice is checked against the CPU checker."""
    import numpy as np
    from beantensor_b200 import sharding
    from oracle import oracle as O
    Bn, M, N, K = 64, 512, 512, 128
    total_batch = Bn * world if weak else Bn
    lo, hi = sharding.batch_slice(total_batch, rank, world)
    nb = hi - lo
    per_set = nb * (M * K + K * N + M * N) * 2
    sets = max(2, min(48, (2 * L2_BYTES) // max(per_set, 1) + 1)) if nb else 1
    bufs = []
    for s in range(sets):
        a = synth_f16((max(nb, 1) * M, K), K ** -0.5, 3, 1000 * s + 2 * rank, torch.float16).view(-1, M, K)[:nb].cuda()
        b = synth_f16((max(nb, 1) * K, N), K ** -0.5, 3, 1000 * s + 2 * rank + 1, torch.float16).view(-1, K, N)[:nb].cuda()
        bufs.append((a, b, torch.empty((nb, M, N), dtype=torch.float16, device="cuda")))

    def step(i):
        a, b, c = bufs[i % sets]
        ops.bmm_gpu(a, b, c)

    us = time_graph(torch, step, sets, steps, 5) if nb else 0.0
    ops.check_device_status(torch.cuda.current_device())
    t = torch.tensor([us], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us_max = float(t.item())
    err = 0.0
    if nb:
        a, b, c = bufs[0]
        c.fill_(float("nan"))
        ops.bmm_gpu(a, b, c)
        torch.cuda.synchronize()
        chk = min(nb, 4)  # the first products of the slice against the CPU checker
        ref = O.bmm(O.F16, a[:chk].cpu().view(torch.uint16).numpy(), b[:chk].cpu().view(torch.uint16).numpy())
        err = O.rel_frobenius(c[:chk].cpu().view(torch.uint16).numpy(), O.F16, ref)
        if torch.isnan(c).any().item():
            err = float("inf")
    e = torch.tensor([err], dtype=torch.float64, device="cuda")
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    err_max = float(e.item())
    algo = total_batch * (M * K + K * N + M * N) * 2
    gbs = algo / (us_max * 1e-6) / 1e9
    return {"workload": f"batched fp16 matmul [{total_batch},512,128]x[{total_batch},128,512] sharded by batch index over {world} ranks, "
                        f"no collective ({'weak: 64 products per rank' if weak else 'strong: 64 products in all'})",
            "us_per_step": us_max, "value": gbs, "unit": "GB/s", "tflops": 2.0 * total_batch * M * N * K / (us_max * 1e-6) / 1e12,
            "scaling": "weak" if weak else "strong", "launch": f"CUDA graph of {sets} launches per rank, replayed; max over ranks",
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peaks["hbm_gbs"], "unit": "GB/s per GPU",
                         "frac": gbs / world / peaks["hbm_gbs"], "traffic": None},
            "parity_check": {"products_per_rank": min(nb, 4), "rel_frob_max_over_ranks": err_max, "tolerance": 2e-3, "ok": err_max <= 2e-3}}


def run_multi(args, peaks):
    import ctypes as C
    import numpy as np
    import torch
    import torch.distributed as dist
    from beantensor_b200 import _lib, ops, sharding
    from beantensor_b200.errors import raise_for_status
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ops.init(local_rank)
    L = _lib.lib()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to come up: start it before the inputs are built
    n = 16384
    c_lo, c_hi = sharding.column_block(n, rank, world)
    nloc = c_hi - c_lo
    dtype = torch.bfloat16
    flops = 2.0 * n ** 3
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    # A lives in shared (peer-addressable) memory too: the end-to-end leg uploads one row panel per rank and
    # replicates it over NVLink instead of pushing all of A through every rank's PCIe link.
    a_buf = SharedBuffer(L, dist, local_rank, rank, world, n * n * 2)
    c_buf = SharedBuffer(L, dist, local_rank, rank, world, n * n * 2)
    a = _wrap_device_memory(torch, a_buf.ptr.value, (n, n)).view(dtype)
    c_dev = _wrap_device_memory(torch, c_buf.ptr.value, (n, n)).view(dtype)
    a.copy_(synth_f16((n, n), n ** -0.5, 4, 0, dtype))
    b_block = synth_f16((n, nloc), n ** -0.5, 4, 1 + rank, dtype).cuda()

    # ---- the same product on one GPU, in this run, every rank at once (the baseline of the efficiency figure)
    b_full = torch.empty((n, n), dtype=dtype, device="cuda")
    for r in range(world):
        b_full[:, r * nloc:(r + 1) * nloc] = synth_f16((n, nloc), n ** -0.5, 4, 1 + r, dtype).cuda()
    c_one = torch.empty((n, n), dtype=dtype, device="cuda")
    one_ms, _, _ = time_reps(torch, dist, world, lambda i: ops.matmul_gpu(a, b_full, c_one), 3, 3, 0.15, 20)
    t1_ms = statistics.median(one_ms) / 3  # max over ranks per region, median region
    ref_sum = checksum(torch, c_one)       # the one-GPU product of the same inputs, for the cross-check below
    del b_full
    torch.cuda.empty_cache()

    # ---- the sharded product with the all-gather fused into the epilogue. Two forms of the peer leg: multimem stores
    # to an NVSwitch multicast mapping of C (one outbound copy per tile; used when every rank's device supports it), or
    # plain stores to each peer's copy in turn. The one that is not timed as the headline is timed as a comparator.
    from beantensor_b200 import multicast
    mcb, mc_note = None, None
    if not args.no_multicast:
        try:
            mcb = multicast.MulticastBuffer(dist, local_rank, rank, world, n * n * 2)
        except NotImplementedError as e:
            mc_note = str(e)
    else:
        mc_note = "switched off by --no-multicast"

    def step_peer(i):
        raise_for_status(L.btm_gemm_nshard(local_rank, stream, _lib.BF16, n, nloc, n, a.data_ptr(), n, b_block.data_ptr(), nloc,
                                           c_buf.table, n, rank, world))

    def step_mc(i):
        raise_for_status(L.btm_gemm_nshard_mc(local_rank, stream, _lib.BF16, n, nloc, n, a.data_ptr(), n, b_block.data_ptr(), nloc,
                                              mcb.local_ptr, mcb.mc_ptr, n, rank, world))

    step = step_mc if mcb is not None else step_peer
    if mcb is not None:
        c_dev = _wrap_device_memory(torch, mcb.local_ptr, (n, n)).view(dtype)
    collective = "multimem stores to an NVSwitch multicast mapping of C" if mcb is not None else "plain stores to every peer's copy of C"

    ms_list, t0, t1 = time_reps(torch, dist, world, step, args.steps, args.warmup, args.min_span, 100)
    ops.check_device_status(local_rank)
    clocks = sampler.summary(t0, t1) if rank == 0 else None
    sp = spread(ms_list, args.steps)
    ms_step = sp["ms_per_step_median"]
    tflops = flops / (ms_step * 1e-3) / 1e12
    other = None
    if mcb is not None:
        o_ms, _, _ = time_reps(torch, dist, world, step_peer, 5, 3, 0.1, 20)
        other = {"what": "the same product with plain peer stores instead of multimem stores", "ms_per_step": statistics.median(o_ms) / 5}

    # ---- parity of the gathered C (outside the timed region): a fresh product into a cleared C
    c_dev.fill_(float("nan"))
    torch.cuda.synchronize()
    dist.barrier()
    step(0)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    mine = checksum(torch, c_dev)
    lo_hi = torch.stack([mine, -mine])
    dist.all_reduce(lo_hi, op=dist.ReduceOp.MIN)
    ranks_equal = bool(lo_hi[0].item() == -lo_hi[1].item())
    same_as_one_gpu = bool(mine.item() == ref_sum.item())  # bit-equal to the unsharded product on this GPU
    has_nan = bool(torch.isnan(c_dev).any().item())
    rows = [0, 1, 127, 128, 4999, 8191, 12345, n - 1]
    rel = None
    if rank == 0:
        from oracle import oracle as O
        a_rows = a[rows].cpu().view(torch.uint16).numpy()
        num = den = 0.0
        for r in range(world):
            b_r = synth_f16((n, nloc), n ** -0.5, 4, 1 + r, dtype).view(torch.uint16).numpy()
            ref = O.gemm(O.BF16, a_rows, b_r)
            got = O.widen(c_dev[rows][:, r * nloc:(r + 1) * nloc].cpu().contiguous().view(torch.uint16).numpy(), O.BF16)
            num += float(((got - ref) ** 2).sum())
            den += float((ref ** 2).sum())
        rel = math.sqrt(num / den)
    parity_ok = ranks_equal and not has_nan and (rel is None or rel <= 2e-3)
    parity = {"rows": len(rows), "rel_frob": rel, "tolerance": 2e-3, "ranks_equal": ranks_equal,
              "equals_one_gpu_product_bitwise": same_as_one_gpu, "nan": has_nan, "ok": parity_ok,
              "what": "rank 0 compares the sampled rows of its gathered C with the CPU checker; every rank's checksum of the whole C "
                      "is compared through an all-reduce and with the one-GPU product of the same inputs"}

    # ---- comparator: the same job with an NCCL all-gather (shard product, all_gather_into_tensor, re-layout)
    stage = torch.empty((n, nloc), dtype=dtype, device="cuda")
    gathered = torch.empty((world, n, nloc), dtype=dtype, device="cuda")
    c_nccl = c_one  # reuse

    def nccl_step(i):
        ops.matmul_gpu(a, b_block, stage)
        dist.all_gather_into_tensor(gathered, stage)
        c_nccl.view(n, world, nloc).copy_(gathered.permute(1, 0, 2))

    nccl_ms, _, _ = time_reps(torch, dist, world, nccl_step, 5, 3, 0.1, 20)
    nccl_ms_step = statistics.median(nccl_ms) / 5
    nccl_equal = bool(checksum(torch, c_nccl).item() == mine.item())
    shard_ms, _, _ = time_reps(torch, dist, world, lambda i: ops.matmul_gpu(a, b_block, stage), 5, 3, 0.1, 20)
    shard_ms_step = statistics.median(shard_ms) / 5
    comparator = {"what": "shard product (this library) + torch.distributed all_gather_into_tensor (NCCL) + re-layout copy; comparator, not the product",
                  "ms_per_step": nccl_ms_step, "fused_over_nccl_speedup": nccl_ms_step / ms_step, "result_equals_fused_bitwise": nccl_equal,
                  "shard_product_alone_ms": shard_ms_step, "exposed_collective_ms_fused": ms_step - shard_ms_step}
    del stage, gathered, c_one
    torch.cuda.empty_cache()

    # ---- end to end: every rank uploads its row panel of A and its column block of B, the panels are replicated
    # over NVLink, the product runs, and every rank downloads its own column block of C.
    r_lo, r_hi = rank * (n // world), (rank + 1) * (n // world)
    ha = a[r_lo:r_hi].cpu().pin_memory()
    hb = b_block.cpu().pin_memory()
    hc = torch.empty((n, nloc), dtype=dtype).pin_memory()
    panel_bytes = (r_hi - r_lo) * n * 2

    def e2e_step(i):
        a[r_lo:r_hi].copy_(ha, non_blocking=True)
        b_block.copy_(hb, non_blocking=True)
        raise_for_status(L.btm_replicate_rows(local_rank, stream, a_buf.table, rank, world, r_lo * n * 2, panel_bytes))
        stream_barrier(torch, dist, flag)   # every rank's panel has landed in this rank's A
        step(i)
        stream_barrier(torch, dist, flag)   # every peer's tiles have landed in this rank's C
        hc.copy_(c_dev[:, c_lo:c_hi], non_blocking=True)

    e2e_steps = 5
    e2e_ms, _, _ = time_region(torch, dist, world, e2e_step, e2e_steps, 2)
    e2e_tflops = flops / (e2e_ms / e2e_steps * 1e-3) / 1e12
    got_block = hc.view(torch.uint16)
    e2e_ok = bool(torch.equal(got_block, c_dev[:, c_lo:c_hi].cpu().view(torch.uint16)))

    # ---- two sharded products in a row, whole against pipelined by row panels (GEMM -> all-gather -> next GEMM)
    from beantensor_b200.pipeline import TwoLayerNShard
    b2_block = synth_f16((n, nloc), n ** -0.5, 4, 100 + rank, dtype).cuda()
    c2 = torch.empty((n, nloc), dtype=dtype, device="cuda")
    # panels: as many as still leave each panel of layer 1 about two waves of 256 x 256 tiles on 74 CTA pairs
    panels = 2
    while panels * 2 <= 16 and (n // (panels * 2) // 256) * (nloc // 256) >= 148:
        panels *= 2
    chain = TwoLayerNShard(dist, local_rank, rank, world, _lib.BF16, a, b_block, b2_block,
                           mcb.local_ptr if mcb is not None else None, mcb.mc_ptr if mcb is not None else None,
                           None if mcb is not None else c_buf.peers, c_dev, c2, panels=panels)
    seq_ms, _, _ = time_reps(torch, dist, world, lambda i: chain.run_sequential(), 3, 2, 0.1, 10)
    c2_seq = c2.clone()
    pipe_ms, _, _ = time_reps(torch, dist, world, lambda i: chain.run_pipelined(), 3, 2, 0.1, 10)
    ops.check_device_status(local_rank)
    two_layer = {"what": "C2[:, block] = (A . B1) . B2[:, block]: layer 1 N-sharded with fused all-gather, layer 2 on the gathered C1; "
                         f"two whole products with a barrier between them against {panels} row panels on three streams",
                 "sequential_ms": statistics.median(seq_ms) / 3, "pipelined_ms": statistics.median(pipe_ms) / 3,
                 "speedup": statistics.median(seq_ms) / statistics.median(pipe_ms),
                 "results_equal_bitwise": bool(torch.equal(c2.view(torch.int16), c2_seq.view(torch.int16)))}
    del b2_block, c2, c2_seq, chain
    torch.cuda.empty_cache()

    # ---- batch-sharded batched matmul (no collective)
    bmm_records = [bench_bmm_sharded(torch, dist, ops, rank, world, peaks, 200, weak=False),
                   bench_bmm_sharded(torch, dist, ops, rank, world, peaks, 200, weak=True)]

    ok = parity_ok and all(r["parity_check"]["ok"] for r in bmm_records)
    if rank == 0:
        sampler.stop()
        roof = tensor_roofline(peaks, tflops / world, t1 - t0, clocks)
        roof["unit"] = "TFLOP/s per GPU"
        roof["traffic"] = None
        line = {
            "metric": METRIC_MULTI, "value": tflops, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded 4096^2 blocks tiled)",
            "config": {"workload": workload_multi(world), "collective": collective, "multicast_note": mc_note, "l2": "inputs (1 GiB+) exceed L2", "parallelism": f"nshard{world}",
                       "timing": f"{sp['regions']} regions of exactly {args.steps} steps back to back, max over ranks per region; value is the "
                                 "median region"},
            "timing": sp,
            "t1_ms_same_run": t1_ms,
            "efficiency": t1_ms / (world * ms_step),
            "efficiency_note": "t1_ms_same_run / (n_gpus * ms_per_step): the same 16384^3 product on one GPU (all ranks at once, max over "
                               "ranks, median region) in this run; the N=1 line of this benchmark times another workload (fp16 4096^3)",
            "parity_check": parity,
            "roofline": roof,
            "nccl_comparator": comparator,
            "peer_store_comparator": other,
            "two_layer_pipeline": two_layer,
            "cpu_baseline": None,
            "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": panel_bytes + n * nloc * 2, "d2h_bytes_per_step": n * nloc * 2,
                    "steps": e2e_steps, "bytes_are": "per rank", "result_checked": e2e_ok,
                    "how": "per rank: upload own row panel of A and own column block of B, replicate the panel to the peers over "
                           "NVLink, product with fused all-gather, download own column block of C"},
            "gpu_launches": args.steps * sp["regions"],
            "clocks": clocks,
            "configs": bmm_records,
        }
        print(json.dumps(line), flush=True)
    if mcb is not None:
        mcb.release()
    c_buf.release()
    a_buf.release()
    dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity check failed: " + json.dumps(parity))


class _RawCuda:
    """Zero-copy view of library-owned device memory for torch (CUDA array interface, 16-bit words)."""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i2", "data": (int(ptr), False), "version": 2}


def _wrap_device_memory(torch, ptr, shape):
    return torch.as_tensor(_RawCuda(ptr, shape), device="cuda")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline-only", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--force-kernel", default=None, choices=["1cta", "2cta"],
                    help="pin the 16-bit matmul to the one-CTA or the two-SM kernel (default: the library chooses)")
    ap.add_argument("--size", type=int, default=4096, help="M=N=K of the headline product (profiling aid; the metric is quoted at 4096)")
    ap.add_argument("--no-multicast", action="store_true", help="N > 1: keep the all-gather on plain peer stores")
    ap.add_argument("--min-span", type=float, default=0.6,
                    help="seconds the repeated timed regions should cover, so that clock samples fall inside (0: one region)")
    args = ap.parse_args()
    _, _, world = dist_env()
    if args.force_kernel:
        os.environ["BTM_FORCE_KERNEL"] = args.force_kernel
    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 5
        args.warmup = args.warmup if args.warmup is not None else 1
        run_reference_arm(args)
        return
    multi = world > 1 or args.gpus > 1
    if args.steps is None:
        args.steps = 20 if multi else 200
    if args.warmup is None:
        args.warmup = 3 if multi else 20
    args.warmup = max(args.warmup, 3)
    peaks = load_peaks()
    if multi:
        if world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run); WORLD_SIZE={world}")
        run_multi(args, peaks)
    else:
        run_single(args, peaks)


if __name__ == "__main__":
    main()
