#!/usr/bin/env python
"""Benchmark of the speculative-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload step|gemv|sweep|tp_gemv|prefill|generate] [--impl reference]

Prints ONE JSON line on rank 0.  Workloads:
  step   (default) accepted tokens/s of the 27B-shape speculative decode step: 64-layer random-init
         hybrid, MTP k=3, batch 8, context 8192; a step is k draft passes + one 32-row verify pass +
         acceptance + commit, replayed as one CUDA graph.  The roofline object is for the dominant
         kernel (the tcgen05 W4A16 linear): the step's linear launches replayed alone and event-timed.
  gemv   the INT4-G128 W4A16 GEMV/skinny-GEMM at the 27B layer shapes (default: M=1, 5120->17408,
         the shape the reference quotes its GEMV bandwidth on); a step is `--launches` back-to-back
         launches rotating over distinct weight buffers whose total exceeds twice the L2, so every
         launch streams its weights from HBM.
  sweep  prints a table of every (shape, M) of the MTP-verify sweep to stderr and the M=1 line as JSON.

`value` is GB/s of algorithmic bytes (weights + scales + activations + outputs, each once) with the
inputs resident in HBM; `e2e` is the same metric through the C-ABI call with HOST activations and a
HOST result, both copies inside the timed region.  `--impl reference` times the CPU oracle port of
the reference's linear_int4_naive on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYER_SHAPES = {"q": (5120, 6144), "kv": (5120, 1024), "o": (6144, 5120), "gate_up": (5120, 17408),
                "down": (17408, 5120), "q_gate": (5120, 12288), "gdn_qkv": (5120, 10240), "lm_head": (5120, 151936)}
L2_BYTES = 126 * 1024 * 1024


# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes of w4a16_tc_kernel, from the ncu capture
# summarised under profiles/ (the kernel reads every weight byte once).
NCU_TRAFFIC_RATIO = 0.98


def alg_bytes(M, K, N, out_bytes=2):
    """weights + scales read once, fp16 activations read once, output written once."""
    return N * K // 2 + N * (K // 128) * 2 + M * K * 2 + M * N * out_bytes


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def synth(M, K, N, seed):
    rng = np.random.default_rng(seed)
    W = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)  # uniform nibbles = int4 uniform in [-8, 7]
    S = (np.abs(rng.normal(0.0, 0.02, size=(N, K // 128))) / 7.0).astype(np.float16)
    X = rng.normal(0.0, 1.0, size=(M, K)).astype(np.float16)
    return X, W, S


def reduce_over_ranks(maxima, sums, device="cpu"):
    """Whole-job aggregation for N > 1 (one process per GPU): element-wise MAX of `maxima` (timings: the job
    is as slow as its slowest rank) and SUM of `sums` (units processed) over all ranks.  Works on any
    torch.distributed backend; returns the inputs unchanged when there is a single process."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(maxima), list(sums)
    tmax = torch.tensor(list(maxima), dtype=torch.float64, device=device)
    tsum = torch.tensor(list(sums), dtype=torch.float64, device=device)
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    return tmax.tolist(), tsum.tolist()


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.reader = None

    def start(self):
        import threading
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line)
        self.reader = threading.Thread(target=pump, daemon=True)
        self.reader.start()

    def samples(self):
        """Samples received so far (nvidia-smi takes a few hundred ms to deliver its first one on a box with many
        GPUs: a caller whose timed region is shorter keeps the same load running until one has arrived)."""
        return len(self.lines)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.reader is not None:
            self.reader.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for line in list(self.lines):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(M, K, N, budget_s=12.0):
    """The oracle's port of the reference's linear_int4_naive (fp32, k ascending), OpenMP over N on
    all host cores; bounded sample of the same workload."""
    import oracle
    X, W, S = synth(M, K, N, 0)
    Xf = X.astype(np.float32)
    oracle.linear_int4_naive_f32(Xf, W, S)
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 5 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        oracle.linear_int4_naive_f32(Xf, W, S)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": alg_bytes(M, K, N) / med / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{len(times)} runs of one M={M} K={K} N={N} GEMV (linear_int4_naive port, OpenMP over N), median"}


def run_reference_arm(args, workload_cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M, K, N = workload_cfg["M"], workload_cfg["K"], workload_cfg["N"]
    import oracle
    X, W, S = synth(M, K, N, 0)
    Xf = X.astype(np.float32)
    for _ in range(max(1, args.warmup)):
        oracle.linear_int4_naive_f32(Xf, W, S)
    reps_per_step = 4
    t0 = time.perf_counter()
    for _ in range(args.steps * reps_per_step):
        oracle.linear_int4_naive_f32(Xf, W, S)
    dt = time.perf_counter() - t0
    val = alg_bytes(M, K, N) * args.steps * reps_per_step / dt / 1e9
    line = {
        "impl": "reference", "metric": "int4_gemv_hbm_gbs", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights, fp32 accumulate", "data": "synthetic",
        "config": workload_cfg,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
                         "sample": f"{reps_per_step} GEMVs per step of the oracle's linear_int4_naive port on the host cores"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def gemv_bench(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import xinfer_b200.ops as ops
    from xinfer_b200 import lib
    assert lib().xinfer_b200_init(local_rank) == 0, lib().xinfer_last_cuda_error()

    K, N = LAYER_SHAPES[args.shape]
    M = args.m
    out_bytes = 4 if args.shape == "lm_head" else 2
    out_dtype = torch.float32 if out_bytes == 4 else torch.float16
    per_launch = alg_bytes(M, K, N, out_bytes)
    w_bytes = N * K // 2 + N * (K // 128) * 2
    n_buf = max(2, -(-2 * L2_BYTES // w_bytes) + 1)
    X, W, S = synth(M, K, N, 0)
    Xd = torch.from_numpy(X).cuda()
    Ws = [torch.from_numpy(np.roll(W, i, axis=0)).cuda() for i in range(n_buf)]
    Ss = [torch.from_numpy(np.roll(S, i, axis=0)).cuda() for i in range(n_buf)]
    Y = torch.empty((M, N), dtype=out_dtype, device="cuda")
    launches = args.launches
    stream = torch.cuda.current_stream()

    def step():
        for i in range(launches):
            j = i % n_buf
            ops.linear_int4(Y, Xd, Ws[j], Ss[j], None, M, N, K)

    # the inner loop is launch-bound for small shapes: capture it once, as the decode graph does
    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(max(3, args.warmup)):
        graph.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        graph.replay()
    ev1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert ops.device_status(local_rank) == 0
    path = ops.last_linear_path()
    total_launches = args.steps * launches
    per_launch_s = ms * 1e-3 / total_launches
    gbs_per_gpu = per_launch / per_launch_s / 1e9
    value = gbs_per_gpu * world

    # end to end: host activations in pinned memory -> C-ABI call -> host result, every launch
    Xh = torch.from_numpy(X).pin_memory()
    Yh = torch.empty((M, N), dtype=out_dtype).pin_memory()
    e2e_launches = min(total_launches, 2000)
    for _ in range(20):
        Xd.copy_(Xh, non_blocking=True)
        ops.linear_int4(Y, Xd, Ws[0], Ss[0], None, M, N, K)
        Yh.copy_(Y, non_blocking=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_launches):
        j = i % n_buf
        Xd.copy_(Xh, non_blocking=True)
        ops.linear_int4(Y, Xd, Ws[j], Ss[j], None, M, N, K)
        Yh.copy_(Y, non_blocking=True)
        stream.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = per_launch * e2e_launches / e2e_s / 1e9 * world

    peak, peak_kind = measured_peak()
    line = {
        "metric": "int4_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"INT4-G128 W4A16 linear M={M} K={K} N={N} ({args.shape}), {launches} launches/step "
                               f"in one CUDA graph", "M": M, "K": K, "N": N,
                   "l2": f"rotates over {n_buf} distinct weight buffers ({n_buf * w_bytes >> 20} MiB > 2x L2)",
                   "kernel_path": {1: "tcgen05", 2: "cuda-core", 3: "tcgen05 gemm (M > 32)"}.get(path, "none")},
        "roofline": {"bound": "hbm", "achieved": gbs_per_gpu, "peak": peak, "unit": "GB/s", "frac": gbs_per_gpu / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_nominal_8000": gbs_per_gpu / 8000.0,
                     "traffic": NCU_TRAFFIC_RATIO * per_launch,
                     "bytes_per_launch": per_launch, "us_per_launch": per_launch_s * 1e6},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": M * K * 2 * launches,
                "d2h_bytes_per_step": M * N * out_bytes * launches, "us_per_call": e2e_s / e2e_launches * 1e6},
        "gpu_launches": total_launches, "clocks": clocks,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(M, K, N)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def prefill_bench(args):
    """One prefill chunk (M = --rows, default 512) through the linears of one Gated-DeltaNet layer and one attention
    layer of the 27B shape, i.e. the `M > 32` side of the same entry points: useful TFLOP/s (2*M*N*K per projection)
    against the measured dense bf16 peak.  The kernel feeds scale * weight to the MMA as an exact hi + lo pair, so
    the tensor pipe does twice the useful work; `roofline.frac` counts useful flops only."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import xinfer_b200.ops as ops
    from xinfer_b200 import lib
    assert lib().xinfer_b200_init(local_rank) == 0, lib().xinfer_last_cuda_error()
    M = args.m if args.m > 32 else 512
    H, F = 5120, 17408
    rng = np.random.default_rng(0)

    def weights(K, N):
        W = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
        S = (np.abs(rng.normal(0, 0.02, size=(N, K // 128))) / 7).astype(np.float16)
        return torch.from_numpy(W).cuda(), torch.from_numpy(S).cuda()

    X = torch.randn((M, H), device="cuda").half()
    Xo = torch.randn((M, 6144), device="cuda").half()
    Xf = torch.randn((M, F), device="cuda").half()
    projs = {n: weights(H, n) for n in (10240, 6144, 48, 12288, 1024)}
    w48b, w1024b = weights(H, 48), weights(H, 1024)
    w_out, w_o = weights(6144, H), weights(6144, H)
    w_gate, w_up, w_down = weights(H, F), weights(H, F), weights(F, H)
    outs = {n: torch.empty((M, n), dtype=torch.float16, device="cuda") for n in (10240, 6144, 48, 12288, 1024, H, F)}
    o48b = torch.empty((M, 48), dtype=torch.float16, device="cuda")
    o1024b = torch.empty((M, 1024), dtype=torch.float16, device="cuda")
    flops = 0

    def d(y, ws, n):
        return {"Y": y, "W_int4": ws[0], "scales": ws[1], "bias": None, "N": n}

    def chunk():
        # Gated-DeltaNet layer: in-projection (4 outputs), out-projection, gate/up + SwiGLU, down
        ops.linear_int4_fused(X, [d(outs[10240], projs[10240], 10240), d(outs[6144], projs[6144], 6144),
                                  d(outs[48], projs[48], 48), d(o48b, w48b, 48)], M, H)
        ops.linear_int4(outs[H], Xo, w_out[0], w_out[1], None, M, H, 6144)
        ops.mlp_gate_up_swiglu_int4(outs[F], X, w_gate[0], w_gate[1], w_up[0], w_up[1], M, F, H)
        ops.linear_int4(outs[H], Xf, w_down[0], w_down[1], None, M, H, F)
        # attention layer: q+gate / k / v, o-projection, the same MLP
        ops.linear_int4_fused(X, [d(outs[12288], projs[12288], 12288), d(outs[1024], projs[1024], 1024),
                                  d(o1024b, w1024b, 1024)], M, H)
        ops.linear_int4(outs[H], Xo, w_o[0], w_o[1], None, M, H, 6144)
        ops.mlp_gate_up_swiglu_int4(outs[F], X, w_gate[0], w_gate[1], w_up[0], w_up[1], M, F, H)
        ops.linear_int4(outs[H], Xf, w_down[0], w_down[1], None, M, H, F)

    flops = 2.0 * M * (H * (10240 + 6144 + 96) + 6144 * H + 2 * H * F + F * H
                       + H * (12288 + 2048) + 6144 * H + 2 * H * F + F * H)
    launches_per_chunk = 4 + 1 + 1 + 1 + 3 + 1 + 1 + 1
    stream = torch.cuda.Stream()
    steps, warm = args.steps, max(3, args.warmup)
    with torch.cuda.stream(stream):
        for _ in range(warm):
            chunk()
        stream.synchronize()
        assert ops.last_linear_path() == 3, "the M > 32 path did not run"
        if world > 1:
            dist.barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(steps):
            chunk()
        ev1.record(stream)
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        extra = 0
        while sampler.samples() == 0 and sampler.proc is not None and extra < 200:
            chunk()
            stream.synchronize()
            extra += 1
        clocks = sampler.stop()
        # end to end: the chunk's activations from pinned host memory, the last projection's output back
        Xh = X.cpu().pin_memory()
        Yh = torch.empty((M, H), dtype=torch.float16).pin_memory()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            X.copy_(Xh, non_blocking=True)
            chunk()
            Yh.copy_(outs[H], non_blocking=True)
            stream.synchronize()
        e2e_s = time.perf_counter() - t0
    assert ops.device_status(local_rank) == 0
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0].item()), float(t[1].item())
    tf_gpu = flops * steps / (ms * 1e-3) / 1e12
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    line = {
        "metric": "prefill_w4a16_gemm_tflops", "value": tf_gpu * world, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"one prefill chunk of M={M} rows through the linears of one Gated-DeltaNet and one "
                               f"attention layer of the 27B shape (hidden 5120, FFN 17408, INT4-G128): "
                               f"{launches_per_chunk} launches, {flops / 1e9:.0f} GFLOP useful", "M": M,
                   "l2": "1.1 GB of distinct weights per chunk (> 2x L2)"},
        "roofline": {"bound": "tensor", "achieved": tf_gpu, "peak": peak, "unit": "TFLOP/s", "frac": tf_gpu / peak,
                     "peak_kind": "of measured (sustained cuBLAS bf16)" if peaks else "of fallback", "traffic": None,
                     "note": "useful flops; the kernel issues two MMAs per k step (exact hi + lo split of scale * weight)"},
        "e2e": {"value": flops * steps / e2e_s / 1e12 * world, "unit": "TFLOP/s", "h2d_bytes_per_step": M * H * 2,
                "d2h_bytes_per_step": M * H * 2},
        "gpu_launches": steps * launches_per_chunk, "clocks": clocks,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def tp_gemv_bench(args):
    """N-split tensor-parallel form of one projection: every rank streams 1/g of the weight rows with the same
    kernel, then one NCCL all-gather restores the [M, N] activation on every rank.  value = whole-projection
    algorithmic bytes per (max over ranks) time; the compute-only time is reported beside it."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import xinfer_b200.ops as ops
    from xinfer_b200 import lib
    from xinfer_b200.tp import ColumnShardedLinear, shard_rows
    assert lib().xinfer_b200_init(local_rank) == 0, lib().xinfer_last_cuda_error()

    K, N = LAYER_SHAPES[args.shape]
    M = args.m
    n0, n1 = shard_rows(N, world, rank)
    X, W, S = synth(M, K, N, 0)
    Wl, Sl = W[n0:n1], S[n0:n1]
    per_launch = alg_bytes(M, K, N, 2)
    slice_bytes = Wl.nbytes + Sl.nbytes
    n_buf = max(2, -(-2 * L2_BYTES // slice_bytes) + 1)
    Xd = torch.from_numpy(X).cuda()
    lins = [ColumnShardedLinear(torch.from_numpy(np.roll(Wl, i, axis=0)).cuda(), torch.from_numpy(np.roll(Sl, i, axis=0)).cuda(),
                                None, N, K, rank=rank, world=world, sliced=True) for i in range(n_buf)]
    Y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    launches = args.launches

    def run(gather):
        for i in range(launches):
            lin = lins[i % n_buf]
            lin.compute_local(Xd, M)
            if gather:
                lin.unstage(lin.gather(M), Y)

    def timed(gather):
        run(gather)
        torch.cuda.synchronize()
        graph = None
        try:  # the launch loop as one CUDA graph (NCCL is capturable); eager if the capture is refused
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                run(gather)
            graph = g
        except Exception:
            torch.cuda.synchronize()
        step = graph.replay if graph is not None else (lambda: run(gather))
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, graph is not None

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_c, _ = timed(False)
    ms_g, graphed = timed(True)
    clocks = sampler.stop()
    assert ops.device_status(local_rank) == 0
    total = args.steps * launches
    us_c, us_g = ms_c * 1e3 / total, ms_g * 1e3 / total
    value = per_launch / (us_g * 1e-6) / 1e9
    peak, peak_kind = measured_peak()
    line = {
        "metric": "int4_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_g / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"INT4-G128 W4A16 linear M={M} K={K} N={N} ({args.shape}), N-split over {world} GPU(s) + "
                               f"all-gather of [M,N] fp16, {launches} launches/step" + (" in one CUDA graph" if graphed else ", eager"),
                   "M": M, "K": K, "N": N, "parallelism": f"tp{world}",
                   "l2": f"rotates over {n_buf} distinct weight shards ({n_buf * slice_bytes >> 20} MiB > 2x L2 per GPU)"},
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak * world, "unit": "GB/s", "frac": value / (peak * world),
                     "peak_kind": f"of {peak_kind} x {world} GPUs", "traffic": None, "us_per_launch": us_g,
                     "us_per_launch_compute_only": us_c,
                     "gbs_compute_only": per_launch / (us_c * 1e-6) / 1e9},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "device-resident operands; the end-to-end form of this metric is the gemv workload"},
        "gpu_launches": total, "clocks": clocks,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sweep(args):
    import torch
    import xinfer_b200.ops as ops
    from xinfer_b200 import lib
    torch.cuda.set_device(0)
    assert lib().xinfer_b200_init(0) == 0
    peak, kind = measured_peak()
    rows = []
    for name in ("q", "kv", "o", "gate_up", "down", "q_gate", "gdn_qkv", "lm_head"):
        K, N = LAYER_SHAPES[name]
        out_bytes = 4 if name == "lm_head" else 2
        w_bytes = N * K // 2 + N * (K // 128) * 2
        n_buf = max(2, -(-2 * L2_BYTES // w_bytes) + 1)
        _, W, S = synth(1, K, N, 0)
        Ws = [torch.from_numpy(np.roll(W, i, axis=0)).cuda() for i in range(n_buf)]
        Ss = [torch.from_numpy(np.roll(S, i, axis=0)).cuda() for i in range(n_buf)]
        for M in (1, 2, 4, 8, 16, 32):
            for path in ((1, 2) if M <= 4 else (1,)):
                X = torch.randn((M, K), device="cuda").half()
                Y = torch.empty((M, N), dtype=torch.float32 if out_bytes == 4 else torch.float16, device="cuda")
                ops.set_linear_path(path)
                launches = max(n_buf, 32)
                g = torch.cuda.CUDAGraph()
                for i in range(2):
                    ops.linear_int4(Y, X, Ws[i % n_buf], Ss[i % n_buf], None, M, N, K)
                torch.cuda.synchronize()
                with torch.cuda.graph(g):
                    for i in range(launches):
                        ops.linear_int4(Y, X, Ws[i % n_buf], Ss[i % n_buf], None, M, N, K)
                for _ in range(3):
                    g.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                reps = 5
                for _ in range(reps):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (reps * launches)
                gbs = alg_bytes(M, K, N, out_bytes) / us / 1e3
                rows.append((name, K, N, M, "tcgen05" if path == 1 else "cuda-core", us, gbs, gbs / peak))
                print(f"{name:8s} K={K:6d} N={N:6d} M={M:2d} {rows[-1][4]:9s} {us:9.2f} us {gbs:8.1f} GB/s "
                      f"{gbs / peak * 100:5.1f}% of {kind}", file=sys.stderr, flush=True)
        ops.set_linear_path(0)
        del Ws, Ss
        torch.cuda.empty_cache()
    assert ops.device_status(0) == 0
    return rows


STEP_SHAPES_M32 = [  # (K, N, count per step) of the 27B-shape verify pass, for the CPU sample
    (5120, 12288 + 1024 + 1024, 16), (6144, 5120, 16 + 48), (5120, 10240 + 6144 + 48 + 48, 48),
    (5120, 17408 * 2, 64), (17408, 5120, 64), (5120, 151936, 1)]


def cpu_step_sample(batch, k, budget_s=15.0):
    """CPU arm of the speculative step: the oracle's port of linear_int4_naive (fp32, OpenMP over N) at
    M = batch*(k+1) on a row sample of each distinct projection shape of the 27B stack; the step time is
    the sample time scaled by weight bytes (the path is weight-streaming bound on the CPU as well).
    Tokens per step are taken as `batch` (one bonus token per sequence, what random weights give)."""
    import oracle
    M = batch * (k + 1)
    total_w = sum(K * N // 2 * cnt for K, N, cnt in STEP_SHAPES_M32) * 1.0
    # MTP head: k passes of fc + one full layer + LM head, M = batch rows (counted by bytes only)
    total_w += k * (10240 * 5120 // 2 + 5120 * 14336 // 2 + 6144 * 5120 // 2 + 5120 * 17408 + 17408 * 5120 // 2 +
                    5120 * 151936 // 2)
    rows = 1024
    t_sample, w_sample = 0.0, 0.0
    t_end = time.perf_counter() + budget_s
    reps = 0
    while reps < 1 or time.perf_counter() < t_end:
        for K, N, _ in STEP_SHAPES_M32:
            X, W, S = synth(M, K, min(rows, N), reps)
            Xf = X.astype(np.float32)
            t0 = time.perf_counter()
            oracle.linear_int4_naive_f32(Xf, W, S)
            t_sample += time.perf_counter() - t0
            w_sample += W.size
        reps += 1
    step_s = t_sample * (total_w / w_sample)
    return {"value": batch / step_s, "unit": "tok/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{reps} passes over a {rows}-row sample of each projection shape at M={M} with the oracle's "
                      f"linear_int4_naive port; step time extrapolated by weight bytes "
                      f"({w_sample / reps / 1e6:.0f} MB sampled of {total_w / 1e9:.2f} GB); {batch} tokens per step",
            "extrapolated_step_s": step_s}


def cpu_gemv_and_acceptance(budget_s=6.0):
    """The other two CPU figures beside the step: the config-0 GEMV at full size (the oracle's port of
    linear_int4_naive, OpenMP over N, median of >= 5 runs) and the acceptance oracle (literal restatement of
    speculative_accept_reject, one thread, as the reference runs it on the host) on the acceptance configuration
    (batch 8, k = 3, vocab 151936, stochastic rule at T = 0.7)."""
    import oracle
    K, N = LAYER_SHAPES["gate_up"]
    X, W, S = synth(1, K, N, 0)
    Xf = X.astype(np.float32)
    oracle.linear_int4_naive_f32(Xf, W, S)
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 5 or (time.perf_counter() < t_end and len(times) < 40):
        t0 = time.perf_counter()
        oracle.linear_int4_naive_f32(Xf, W, S)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    B, k, V = 8, 3, 151936
    rng = np.random.default_rng(0)
    target = rng.normal(0, 3, size=(B, k, V)).astype(np.float32)
    toks = rng.integers(0, V, size=(B, k)).astype(np.int64)
    probs = np.full((B, k), 1e-5, np.float32)
    uni = rng.random(size=(B, k)).astype(np.float32)
    acc = []
    for _ in range(5):
        t0 = time.perf_counter()
        for b in range(B):
            oracle.speculative_accept_reject(toks[b], target[b], probs[b], uni[b], inv_temperature=1.0 / 0.7)
        acc.append(time.perf_counter() - t0)
    return {"gemv": {"value": alg_bytes(1, K, N) / med / 1e9, "unit": "GB/s", "us": med * 1e6, "cores": oracle.num_threads(),
                     "sample": f"{len(times)} runs of the full M=1 K={K} N={N} GEMV, median"},
            "acceptance": {"us": statistics.median(acc) * 1e6, "cores": 1,
                           "sample": f"batch {B} x k {k} x vocab {V}, stochastic rule, 5 runs, median"}}


def gemv_object(ops, torch, tp=None, dist=None, shape="gate_up", M=1, launches=64, reps=5):
    """INT4 GEMV HBM GB/s on the shape the metric is quoted on (M = 1, 5120 -> 17408): `launches` launches in one
    CUDA graph rotating over distinct weight buffers (> 2x L2 in total), event-timed.  With a tensor-parallel group
    every rank streams its 1/g of the rows and stores its slice into every rank's output from the kernel's
    epilogue; the figure is then whole-projection bytes over the slowest rank's time."""
    K, N = LAYER_SHAPES[shape]
    world = 1 if tp is None else tp.world
    rank = 0 if tp is None else tp.rank
    nl = N // world
    _, W, S = synth(M, K, N, 0)
    Wl, Sl = W[rank * nl:(rank + 1) * nl], S[rank * nl:(rank + 1) * nl]
    w_bytes = Wl.nbytes + Sl.nbytes
    n_buf = max(2, -(-2 * L2_BYTES // w_bytes) + 1)
    Ws = [torch.from_numpy(np.roll(Wl, i, axis=0)).cuda() for i in range(n_buf)]
    Ss = [torch.from_numpy(np.roll(Sl, i, axis=0)).cuda() for i in range(n_buf)]
    X = torch.randn((M, K), device="cuda").half()
    if tp is None:
        Y = torch.empty((M, N), dtype=torch.float16, device="cuda")
        def launch(j):
            ops.linear_int4(Y, X, Ws[j], Ss[j], None, M, N, K)
    else:
        y_off = tp.alloc(M * N * 2)
        def launch(j):
            tp.linear(y_off, N, rank * nl, X, Ws[j], Ss[j], None, M, nl, K)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(2):
            launch(i % n_buf)
        stream.synchronize()
        if dist is not None:
            dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(launches):
                launch(i % n_buf)
        for _ in range(3):
            g.replay()
        stream.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * launches)
    if dist is not None:
        t = torch.tensor([us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item())
    gbs = alg_bytes(M, K, N) / us / 1e3
    peak, kind = measured_peak()
    return {"shape": f"M={M} K={K} N={N}", "us": us, "value": gbs, "unit": "GB/s", "frac_of_measured": gbs / (peak * world),
            "frac_of_nominal_8000": gbs / (8000.0 * world), "peak_kind": f"of {kind}" + (f" x {world} GPUs" if world > 1 else ""),
            "parallelism": "one GPU" if world == 1 else f"N-split over {world} GPUs, slices stored into every rank's output "
                           "by the GEMM epilogue (peer stores + flags)",
            "l2": f"rotates over {n_buf} distinct weight buffers per GPU"}


def acceptance_object(ops, torch, launches=20, reps=5):
    """Device time of the acceptance configuration: batch 8, k = 3, vocab 151936 fp32 logits, stochastic rule at
    T = 0.7 with device-resident draft probabilities and uniforms; one call = partials kernel + finish kernel."""
    B, k, V = 8, 3, 151936
    logits = [torch.randn((B, k, V), device="cuda") * 3 for _ in range(4)]   # 58 MB in rotation (L2 holds it: noted)
    toks = torch.randint(0, V, (B, k), device="cuda")
    probs = torch.full((B, k), 1e-5, device="cuda")
    uni = torch.rand((B, k), device="cuda")
    out = torch.zeros(B * ops.ACCEPT_RECORD_BYTES, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ops.speculative_accept_reject_batched(toks, logits[0], probs, uni, out, inv_temperature=1.0 / 0.7)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(launches):
                ops.speculative_accept_reject_batched(toks, logits[i % 4], probs, uni, out, inv_temperature=1.0 / 0.7)
        g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * launches)
    bytes_ = B * k * V * 4
    return {"us": us, "logit_bytes": bytes_, "gbs": bytes_ / us / 1e3,
            "config": f"batch {B}, k {k}, vocab {V}, stochastic rule T=0.7; logits rotate over 4 buffers (58 MB, L2-resident)"}


def step_bench(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import xinfer_b200.ops as ops
    from xinfer_b200 import lib
    from xinfer_b200.spec import Shape, SpecDecoder
    assert lib().xinfer_b200_init(local_rank) == 0, lib().xinfer_last_cuda_error()

    from xinfer_b200.tp import TpGroup
    shape = Shape(num_hidden_layers=args.layers)
    B, k, ctx0 = args.batch, args.k, args.context
    # More than one GPU: the SAME job (one batch-B step) with every projection N-split over the ranks and the
    # per-sequence state split by sequence; --parallel replicas runs N independent copies instead.
    use_tp = world > 1 and args.parallel == "tp"
    tp = None
    if use_tp:
        tp = TpGroup(SpecDecoder.exchange_bytes(shape, B, k, world) + (8 << 20))
        dec = SpecDecoder(shape, batch=B, k=k, max_seq=ctx0 + 1024, seed=0, tp=tp)
        dec.reset(ctx0, seed=0)
        dist.barrier()
    else:
        dec = SpecDecoder(shape, batch=B, k=k, max_seq=ctx0 + 1024, seed=rank)
        if args.temperature > 0:
            dec.set_sampling(args.temperature, 12345 + rank)   # stochastic drafting + rejection rule (one GPU per job)
            if args.top_p < 1.0:
                dec.set_top_p(args.top_p)
        dec.reset(ctx0, seed=rank)
    stream = torch.cuda.Stream()
    steps, warm = args.steps, max(3, args.warmup)
    with torch.cuda.stream(stream):
        dec.capture(stream)          # runs one eager step, then records the step as a CUDA graph
        for _ in range(warm):
            dec.step()
        stream.synchronize()
        ctx_before = dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum()
        if world > 1:
            dist.barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(steps):
            dec.step()
        ev1.record(stream)
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        tokens = int(dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum() - ctx_before)   # of the timed steps only
        # the clock record must hold at least one sample taken under this load: keep the same steps running
        # (untimed) until nvidia-smi has delivered one
        extra = 0
        while extra < 400:
            more = 1 if (sampler.samples() == 0 and sampler.proc is not None) else 0
            if world > 1:  # every rank runs the same number of steps (the N-split step needs all of them): rank 0 decides
                flag = torch.tensor([more], device="cuda", dtype=torch.int32)
                dist.broadcast(flag, src=0)
                more = int(flag.item())
            if not more:
                break
            dec.step()
            stream.synchronize()
            extra += 1
        clocks = sampler.stop()
        if extra:
            clocks["note"] = f"first sample arrived during {extra} untimed steps of the same load right after the timed region"
        launches = dec.info(2)

        # the dominant kernel alone: the step's W4A16 launches, same order and weights, event-timed
        dec.enqueue_linears()
        stream.synchronize()
        lin_bytes, lin_launches = dec.info(4), dec.info(5)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            dec.enqueue_linears()
        g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        lin_reps = 5
        for _ in range(lin_reps):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        lin_ms = e0.elapsed_time(e1) / lin_reps

        # end to end through the decoder's public calls: host token ids in, host emitted tokens out
        toks = np.zeros(B, np.int64)
        e2e_steps = max(5, steps)
        ctx_a = dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            dec.set_tokens(toks)                      # H2D: the tokens the server decided to continue from
            dec.step()
            emitted, counts = dec.results()           # D2H + sync: what the server streams to its clients
            toks = emitted[np.arange(B), counts - 1]
        e2e_s = time.perf_counter() - t0
        e2e_tokens = int(dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum() - ctx_a)
    assert ops.device_status(local_rank) == 0
    if tp is not None:
        assert tp.status() == 0, "an inter-rank exchange wait ran out"
    exchanges = dec.info(6)
    if use_tp:
        # one job: every rank holds the same token counts; the job is as slow as its slowest rank
        (ms, e2e_s, lin_ms), _ = reduce_over_ranks([ms, e2e_s, lin_ms], [0], device="cuda")
    else:
        (ms, e2e_s), (tokens, e2e_tokens) = reduce_over_ranks([ms, e2e_s], [tokens, e2e_tokens], device="cuda")
    tokens, e2e_tokens = int(tokens), int(e2e_tokens)
    value = tokens / (ms * 1e-3)
    # the other half of the metric, and the acceptance kernel, on the same GPUs
    gemv = gemv_object(ops, torch, tp=tp, dist=dist if world > 1 and use_tp else None) if (world == 1 or use_tp) else None
    acceptance = acceptance_object(ops, torch) if rank == 0 else None
    replicas = None
    if use_tp and args.with_replicas:
        # the same GPUs as N independent copies of the job (weak scaling), for comparison
        dec.close()
        dec = SpecDecoder(shape, batch=B, k=k, max_seq=ctx0 + 1024, seed=rank)
        dec.reset(ctx0, seed=rank)
        with torch.cuda.stream(stream):
            dec.capture(stream)
            for _ in range(warm):
                dec.step()
            stream.synchronize()
            c0 = dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum()
            dist.barrier()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record(stream)
            for _ in range(steps):
                dec.step()
            r1.record(stream)
            torch.cuda.synchronize()
            rtok = int(dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum() - c0)
        (rms,), (rtok,) = reduce_over_ranks([r0.elapsed_time(r1)], [rtok], device="cuda")
        replicas = {"value": rtok / (rms * 1e-3), "unit": "tok/s", "ms_per_step": rms / steps, "scaling": "weak",
                    "note": f"{world} independent batch-{B} jobs, one per GPU, no inter-GPU traffic"}
    batch_split = None
    if use_tp and args.with_replicas and B % world == 0:
        # the SAME batch-B job with its sequences divided over the GPUs (each rank the whole model and B / N
        # sequences; sequences are independent, so nothing crosses NVLink): strong scaling without a collective
        dec.close()
        Bl = B // world
        dec = SpecDecoder(shape, batch=Bl, k=k, max_seq=ctx0 + 1024, seed=rank)
        dec.reset(ctx0, seed=rank)
        with torch.cuda.stream(stream):
            dec.capture(stream)
            for _ in range(warm):
                dec.step()
            stream.synchronize()
            c0 = dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum()
            dist.barrier()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record(stream)
            for _ in range(steps):
                dec.step()
            r1.record(stream)
            torch.cuda.synchronize()
            btok = int(dec.tensor(-1, "ctx", np.int32).astype(np.int64).sum() - c0)
        (bms,), (btok,) = reduce_over_ranks([r0.elapsed_time(r1)], [btok], device="cuda")
        batch_split = {"value": btok / (bms * 1e-3), "unit": "tok/s", "ms_per_step": bms / steps, "scaling": "strong",
                       "note": f"the same batch-{B} job, {Bl} sequence(s) per GPU, whole model on every GPU, no inter-GPU traffic"}
    peak, peak_kind = measured_peak()
    lin_gbs = lin_bytes / (lin_ms * 1e-3) / 1e9
    line = {
        "metric": "accepted_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong" if use_tp else "weak", "vs_baseline": None,
        "dtype": "int4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"27B-shape hybrid ({args.layers} layers: Gated-DeltaNet + full attention, hidden 5120, "
                               f"FFN 17408, vocab 151936, INT4-G128), MTP k={k}, batch {B}, context {ctx0}, "
                               + ("greedy; " if args.temperature <= 0 or use_tp else f"stochastic at T={args.temperature}" + (f", top-p {args.top_p}" if args.top_p < 1.0 else "") + "; ") +
                               f"one step = {k} MTP draft passes + one {B * (k + 1)}-row verify pass + acceptance + "
                               f"commit, replayed as one CUDA graph",
                   "layers": args.layers, "batch": B, "k": k, "context": ctx0,
                   "parallelism": (f"tp{world}: every projection N-split over {world} GPUs, KV cache and recurrent state split "
                                   f"by sequence, LM head split by vocabulary") if use_tp
                                  else f"{world} independent replica(s), one per GPU",
                   "collective": (f"{exchanges} exchanges per step inside the CUDA graph: the GEMM epilogue stores its slice "
                                  "into every rank's activation buffer with plain peer stores over NVLink, one flag per "
                                  "(receiver, sender), bounded waits; no NCCL on the data path") if use_tp else "none",
                   "l2": "inputs larger than L2: every step streams %.1f GB of weights" % (dec.info(0) / 1e9),
                   "accepted_per_step_per_seq": tokens / max(1, steps * B * (1 if use_tp else world)),
                   "note": "random-init weights: the draft head and the target agree only by chance, so almost "
                           "every step emits the bonus token alone"},
        "roofline": {"bound": "hbm", "achieved": lin_gbs, "peak": peak, "unit": "GB/s", "frac": lin_gbs / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_nominal_8000": lin_gbs / 8000.0,
                     "traffic": NCU_TRAFFIC_RATIO * lin_bytes / max(1, lin_launches),
                     "traffic_source": "ncu dram__bytes_read+write of one gate_up M=32 launch (46.4 MB for 47.4 MB "
                                       "algorithmic), scaled by bytes to the average launch of the step",
                     "kernel": "w4a16_tc_kernel", "launches_per_step": lin_launches,
                     "bytes_per_launch": lin_bytes / max(1, lin_launches),
                     "us_per_launch": lin_ms * 1e3 / max(1, lin_launches), "linears_ms_per_step": lin_ms,
                     "linears_share_of_step": lin_ms / (ms / steps)},
        "e2e": {"value": e2e_tokens / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": B * 8,
                "d2h_bytes_per_step": B * (k + 1) * 8 + B * 4, "ms_per_step": e2e_s / e2e_steps * 1e3},
        "gpu_launches": launches * steps, "clocks": clocks,
    }
    if clocks.get("sm_mhz"):
        # clock-normalised reading: the same step at another SM clock takes about this many ms x MHz / that clock
        line["ms_per_step_x_sm_mhz"] = ms / steps * clocks["sm_mhz"]
    if gemv is not None:
        line["gemv"] = gemv
    if acceptance is not None:
        line["acceptance"] = acceptance
    if replicas is not None:
        line["replicas"] = replicas
    if batch_split is not None:
        line["batch_split"] = batch_split
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_step_sample(B, k)
            line["cpu_baseline"].update(cpu_gemv_and_acceptance())
        print(json.dumps(line), flush=True)
    dec.close()
    if tp is not None:
        dist.barrier()
        tp.close()
    if world > 1:
        dist.destroy_process_group()


def step_reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    B, k = args.batch, args.k
    per = max(2.0, min(20.0, 90.0 / max(1, args.steps + args.warmup)))
    for _ in range(min(1, args.warmup)):
        cpu_step_sample(B, k, budget_s=1.0)
    res = [cpu_step_sample(B, k, budget_s=per) for _ in range(min(args.steps, 5))]
    step_s = statistics.median(r["extrapolated_step_s"] for r in res)
    val = B / step_s
    line = {"impl": "reference", "metric": "accepted_tok_per_s", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            # (the same one batch-B job at every N, as the N-split arm it stands beside; replicas: N such jobs)
            "scaling": "strong" if (args.gpus > 1 and args.parallel == "tp") else "weak", "vs_baseline": None,
            "dtype": "int4 weights, fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"27B-shape hybrid ({args.layers} layers: Gated-DeltaNet + full attention, hidden 5120, "
                                   f"FFN 17408, vocab 151936, INT4-G128), MTP k={k}, batch {B}, context {args.context}, greedy; "
                                   f"one step = {k} MTP draft passes + one {B * (k + 1)}-row verify pass + acceptance + commit",
                       "layers": args.layers, "batch": B, "k": k, "context": args.context,
                       "note": "CPU arm: the oracle's port of the reference's linear_int4_naive on all host cores over a "
                               "bounded row sample of every projection shape; the step time is extrapolated by weight "
                               "bytes (the linears are 88 % of the reference's own step)"},
            "cpu_baseline": dict(res[0], value=val, **cpu_gemv_and_acceptance()),
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def generate_bench(args):
    """One request batch through `xinfer_spec_decoder_generate` (the reference's Engine::generate loop, device side):
    `--batch` prompts of `--prompt-len` synthetic tokens, `--max-new` tokens each, on the 27B shape with the step
    captured as a CUDA graph.  Host buffers in and out; the timers are the call's own (time to first token = reset +
    prefill + first step, decode tokens/s over the steps after it).  One GPU."""
    import torch
    from xinfer_b200 import lib
    from xinfer_b200.spec import Shape, SpecDecoder
    torch.cuda.set_device(0)
    assert lib().xinfer_b200_init(0) == 0, lib().xinfer_last_cuda_error()
    shape = Shape(num_hidden_layers=args.layers)
    B, k, T, cap = args.batch, args.k, args.prompt_len, args.max_new
    dec = SpecDecoder(shape, batch=B, k=k, max_seq=T + cap + 64, seed=0)
    if args.temperature > 0:
        dec.set_sampling(args.temperature, 1234)
        if args.top_p < 1.0:
            dec.set_top_p(args.top_p)
    dec.reset(T, seed=0)
    stream = torch.cuda.Stream()
    prompt = np.random.default_rng(0).integers(0, shape.vocab_size, size=(B, T)).astype(np.int64)
    runs = []
    sampler = ClockSampler(0)
    with torch.cuda.stream(stream):
        dec.capture(stream)
        for i in range(max(1, args.warmup) + max(1, args.steps)):
            if i == max(1, args.warmup):
                sampler.start()
            res = dec.generate(prompt, max_new_tokens=cap, temperature=args.temperature, top_p=args.top_p, seed=1234)
            if i >= max(1, args.warmup):
                runs.append(res)
    clocks = sampler.stop()
    r0 = runs[len(runs) // 2][0]
    med = lambda f: statistics.median(f(r[0]) for r in runs)
    generated = sum(x.generated_tokens for x in runs[-1])
    line = {
        "metric": "accepted tok/s", "value": med(lambda x: x.decode_tokens_per_sec), "unit": "tok/s", "n_gpus": 1,
        "steps": len(runs), "warmup": max(1, args.warmup), "ms_per_step": med(lambda x: x.total_time_sec) * 1e3 / max(1, r0.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int4 x fp16, fp32 accumulate",
        "data": "synthetic", "impl": "ours",
        "config": {"workload": f"generate: {B} prompts x {T} tokens, {cap} new tokens each, 27B-shape hybrid ({args.layers} layers), "
                               f"k={k}, temperature {args.temperature}, top-p {args.top_p}, random-init INT4-G128 weights (no draft is accepted at "
                               "temperature 0: one token per sequence and step)",
                   "batch": B, "k": k, "prompt_len": T, "max_new_tokens": cap},
        "generate": {"time_to_first_token_ms": med(lambda x: x.time_to_first_token_sec) * 1e3,
                     "total_ms": med(lambda x: x.total_time_sec) * 1e3, "steps_per_request": r0.steps,
                     "generated_tokens": generated, "finish": sorted({x.finish_reason for x in runs[-1]}),
                     "prefill_tok_s": B * T / max(1e-9, med(lambda x: x.time_to_first_token_sec)),
                     "note": "prefill runs 512-row chunks (projections on the M = 512 GEMM, each mixer one launch per chunk); the reset that starts a request is inside the first-token time"},
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    dec.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="step", choices=["step", "gemv", "sweep", "tp_gemv", "prefill", "generate"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--temperature", type=float, default=0.0,
                    help="step workload: > 0 runs stochastic drafting and the rejection rule (default 0: greedy, the metric's configuration)")
    ap.add_argument("--prompt-len", type=int, default=64, help="generate workload: prompt tokens per sequence")
    ap.add_argument("--max-new", type=int, default=64, help="generate workload: tokens to generate per sequence")
    ap.add_argument("--top-p", dest="top_p", type=float, default=1.0,
                    help="with --temperature > 0: nucleus sampling on both sides of the rejection rule (default 1: off)")
    ap.add_argument("--shape", default="gate_up", choices=sorted(LAYER_SHAPES))
    ap.add_argument("--m", "--rows", dest="m", type=int, default=1)  # activation rows M (--rows: torchrun parses --m itself)
    ap.add_argument("--launches", type=int, default=64)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallel", default="tp", choices=["tp", "replicas"],
                    help="with more than one GPU: the one job N-split over the GPUs (default), or N independent copies")
    ap.add_argument("--with-replicas", dest="with_replicas", action="store_true", default=True,
                    help="tp runs also measure, on the same GPUs, N independent replicas and the batch divided by sequence (default)")
    ap.add_argument("--no-replicas", dest="with_replicas", action="store_false", help="tp runs measure the N-split only")
    args = ap.parse_args()
    if args.impl == "reference":
        # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every host thread,
        # so restore the default before the OpenMP runtime of the oracle library is loaded
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    K, N = LAYER_SHAPES[args.shape]
    cfg = {"workload": f"INT4-G128 W4A16 linear M={args.m} K={K} N={N} ({args.shape})", "M": args.m, "K": K, "N": N}
    if args.workload == "step":
        if args.impl == "reference":
            step_reference_arm(args)
        else:
            step_bench(args)
        return
    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return
    if args.workload == "tp_gemv":
        return tp_gemv_bench(args)
    if args.workload == "prefill":
        return prefill_bench(args)
    if args.workload == "generate":
        return generate_bench(args)
    if args.workload == "sweep":
        sweep(args)
        return
    gemv_bench(args)


if __name__ == "__main__":
    main()
