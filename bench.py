#!/usr/bin/env python
"""Benchmark of the speculative-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemv|sweep] [--impl reference]

Prints ONE JSON line on rank 0.  Workloads:
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


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
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
                   "kernel_path": {1: "tcgen05", 2: "cuda-core"}.get(path, "none")},
        "roofline": {"bound": "hbm", "achieved": gbs_per_gpu, "peak": peak, "unit": "GB/s", "frac": gbs_per_gpu / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_nominal_8000": gbs_per_gpu / 8000.0, "traffic": None,
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemv", choices=["gemv", "sweep"])
    ap.add_argument("--shape", default="gate_up", choices=sorted(LAYER_SHAPES))
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--launches", type=int, default=64)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    K, N = LAYER_SHAPES[args.shape]
    cfg = {"workload": f"INT4-G128 W4A16 linear M={args.m} K={K} N={N} ({args.shape})", "M": args.m, "K": K, "N": N}
    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return
    if args.workload == "sweep":
        sweep(args)
        return
    gemv_bench(args)


if __name__ == "__main__":
    main()
