#!/usr/bin/env python
"""Benchmark of the fused 4-bit dequant-GEMV path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode7b|e2m1_4096|gf4_11008|decode70b] [--batch B]

A "step" is one decode token of the workload: every matrix of the layer stack
multiplied once by its own activation vector (the reference has no attention,
norm or residual, so the matrices are independent problems).  Default
workload: Llama-2-7B-shaped stack, 32 layers x {q,k,v,o 4096x4096, gate,up
11008x4096, down 4096x11008}, GF4 codes with fp16 group-128 scales, per-row
16-entry Jenks codebooks, 128-wide block-Hadamard-rotated inputs, batch 1,
bf16 activations.  Weights are random-init N(0, 0.02); one matrix per distinct
shape is quantised with the real packer and copied into distinct allocations
for every use, so a token reads 3.39 GB of distinct HBM (far beyond L2).

N > 1 (torchrun, one rank per GPU): every matrix is row-sharded over the
ranks; the output slices reach every rank either by peer stores from the GEMV
epilogue plus a barrier (--exchange fused, the default) or by one NCCL
all-gather per step (--exchange nccl).

Rank 0 prints one JSON line: metric, value, unit, per-step time, clocks seen
during the timed region, the end-to-end figure with host copies (e2e), the
roofline of the dominant kernel, and (N = 1) a CPU baseline.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

HBM_NOMINAL_GBS = 8000.0
# DRAM bytes (read + write) per algorithmic byte of the grouped GEMV kernel, from one ncu capture each on a
# smaller case of the same kernel (profiles/gemv_grouped_gf4_11008x4096.md: 381.93 MB for 378.10 MB;
# profiles/gemv_grouped_e2m1_8192x8192.md: 608.58 MB for 604.50 MB); traffic grows in proportion to the
# rows processed, so a full launch's traffic is this ratio times its algorithmic bytes.
DRAM_TRAFFIC_RATIO = {"gf4": 381.930496 / 378.101760, "e2m1": 608.581888 / 604.504064}

WORKLOADS = {
    # name: (fmt, group, had_block, layers, [(label, N, K, count-per-layer)], init std)
    "decode7b": ("gf4", 128, 128, 32, [("qkvo", 4096, 4096, 4), ("gate_up", 11008, 4096, 2), ("down", 4096, 11008, 1)], 0.02),
    "decode70b": ("e2m1", 32, 0, 80, [("qo", 8192, 8192, 2), ("kv", 1024, 8192, 2), ("gate_up", 28672, 8192, 2),
                                       ("down", 8192, 28672, 1)], 0.015),
    "e2m1_4096": ("e2m1", 32, 0, 16, [("linear", 4096, 4096, 1)], 0.02),
    "gf4_11008": ("gf4", 128, 128, 16, [("linear", 11008, 4096, 1)], 0.02),
    "e2m1_8192": ("e2m1", 32, 0, 16, [("linear", 8192, 8192, 1)], 0.02),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        for l in rows:
            f = [c.strip() for c in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_stack(name: str, rank: int, world: int, batch: int, device, threads: int = 0):
    """Quantise one matrix per distinct shape, shard its rows, and copy the
    shard into a distinct allocation per use.  Returns (weights, meta)."""
    import if_i_could_turn_back_time_b200 as jq
    fmt, g, had, layers, mats, std = WORKLOADS[name]
    spec = jq.QuantSpec(fmt, g, had)
    gen = torch.Generator("cpu").manual_seed({"decode7b": 3, "decode70b": 4, "e2m1_4096": 1, "gf4_11008": 2, "e2m1_8192": 5}[name])
    proto = {}
    t0 = time.time()
    for label, N, K, _ in mats:
        if N % world:
            raise SystemExit(f"N={N} of {label} does not divide over {world} ranks")
        lo, hi = rank * (N // world), (rank + 1) * (N // world)
        W = torch.randn(N, K, generator=gen) * std     # every rank draws the same matrix, keeps its rows
        if fmt == "e2m1":
            W = W.bfloat16().float()
        proto[label] = jq.pack_weight(W[lo:hi].to(device), spec, threads=threads)   # quantised on the GPU
        del W
    pack_s = time.time() - t0
    weights, labels = [], []
    for _layer in range(layers):
        for label, N, K, cnt in mats:
            for _ in range(cnt):
                weights.append(proto[label].to(device))   # .to() copies: a distinct allocation per use
                labels.append(label)
    alg = sum(jq.algorithmic_bytes(spec, w.N, w.K, batch, 2, 2) for w in weights)
    meta = {"spec": spec, "pack_seconds": pack_s, "alg_bytes_rank": alg, "n_matrices": len(weights),
            "weights_total": sum(w.N * w.K for w in weights)}
    return weights, meta


def cpu_reference_leg(name: str, batch: int, budget_s: float, steps: int = 1, warmup: int = 0):
    """Times the reference's forward form (per-call dequantise + fp32 F.linear,
    Quantization_Experiments/layers.py:36-38) on the host cores, on a bounded
    sample of the workload, and scales to tokens/s by weight count."""
    import if_i_could_turn_back_time_b200 as jq
    from oracle import ref_linear
    fmt, g, had, layers, mats, std = WORKLOADS[name]
    spec = jq.QuantSpec(fmt, g, had)
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    label, N, K, _ = mats[0]
    rows = min(N, 1024)   # a row block of the first matrix shape: cost is linear in rows
    gen = torch.Generator("cpu").manual_seed(0)
    pw = jq.pack_weight(torch.randn(rows, K, generator=gen) * std, spec)
    x = torch.randn(batch, K, generator=gen).bfloat16()
    total_w = sum(n * k * c for _, n, k, c in mats) * layers
    call = lambda: ref_linear.per_call(x, pw.qweight, pw.scales, pw.codebook, None, rows, K, g, had)
    call()
    t = time.perf_counter(); call(); one = time.perf_counter() - t
    reps = max(1, min(200, int(budget_s / max(one, 1e-4) / max(1, steps + warmup))))
    times = []
    for i in range(warmup + steps):
        t = time.perf_counter()
        for _ in range(reps):
            call()
        dt = (time.perf_counter() - t) / reps
        if i >= warmup:
            times.append(dt)
    per_weight = statistics.median(times) / (rows * K)
    tok_s = batch / (per_weight * total_w)
    return {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{rows}x{K} row block of '{label}' ({fmt} g{g}), {reps} calls/step, per-call dequant + fp32 "
                      f"F.linear in PyTorch on CPU, scaled by weight count to the {total_w / 1e9:.2f} G-weight stack"}, \
        statistics.median(times) * (total_w / (rows * K))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode7b", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--cpu-budget", type=float, default=15.0, help="seconds of CPU work for the cpu_baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: all-gather fused into the GEMV epilogue (peer stores) or one NCCL all-gather per step")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    fmt, g, had, layers, mats, std = WORKLOADS[args.workload]
    config = {"workload": f"{args.workload}: {layers} layers x " + ", ".join(f"{c}x{n}x{k}" for _, n, k, c in mats) +
                          f", {fmt} g{g}" + (f" + block-Hadamard-{had}" if had else "") + f", batch {args.batch}, bf16 activations",
              "batch": args.batch, "parallelism": f"row-shard x{world} + all-gather" if world > 1 else "single GPU",
              "l2": "inputs larger than L2 (every matrix has its own allocation; one step streams them all once)"}

    if args.impl == "reference":
        if rank != 0:
            return
        cb, step_s = cpu_reference_leg(args.workload, args.batch, 60.0, steps=args.steps, warmup=min(args.warmup, 1))
        line = {"impl": "reference", "metric": "decode tokens/s", "value": cb["value"], "unit": "tok/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from if_i_could_turn_back_time_b200 import ops
    threads = max(1, len(os.sched_getaffinity(0)) // max(1, world))
    weights, meta = build_stack(args.workload, rank, world, args.batch, device, threads)
    exchange = "none"
    grp = None
    if world > 1 and args.exchange == "fused" and args.batch <= 8:
        try:
            grp = ops.GroupedGemv(weights, args.batch, torch.bfloat16, full_rows=[w.N * world for w in weights],
                                  row_offsets=[w.N * rank for w in weights], group=dist.group.WORLD)
            exchange = "fused peer stores + barrier"
        except Exception as e:  # symmetric memory unavailable: fall back to the NCCL exchange
            if rank == 0:
                print(f"fused exchange unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
            grp = None
    if grp is None:
        grp = ops.GroupedGemv(weights, args.batch, torch.bfloat16)
        if world > 1:
            exchange = "nccl all_gather_into_tensor"
    fused = grp.fused_exchange
    gen = torch.Generator("cpu").manual_seed(100)
    x_host = torch.empty(grp.x_arena.numel(), dtype=torch.uint8).pin_memory()
    x_host.view(torch.bfloat16).copy_(torch.randn(grp.x_arena.numel() // 2, generator=gen).bfloat16())
    y_host = torch.empty(grp.y_arena.numel() * (1 if fused else world), dtype=torch.uint8).pin_memory()
    grp.x_arena.copy_(x_host)
    y_all = torch.empty(grp.y_arena.numel() * world, dtype=torch.uint8, device=device) if (world > 1 and not fused) else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    kernel_events = []

    def step(e2e: bool, record: bool = False):
        if e2e:
            grp.x_arena.copy_(x_host, non_blocking=True)
        if record:
            a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
            a.record()
        grp.run()
        if record:
            b.record()
            kernel_events.append((a, b))
        if fused:
            grp.barrier()
        elif world > 1:
            dist.all_gather_into_tensor(y_all, grp.y_arena)
        if e2e:
            src = y_all if y_all is not None else grp.y_arena
            y_host.copy_(src, non_blocking=True)
            torch.cuda.current_stream().synchronize()   # the caller needs the result before the next token

    def timed(e2e: bool, steps: int, warmup: int, record: bool):
        for _ in range(warmup):
            step(e2e)
        barrier()
        t0 = time.time()
        start = torch.cuda.Event(enable_timing=True); end = torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step(e2e, record)
        end.record()
        barrier()
        t1 = time.time()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps, t0, t1

    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    ms_step, t0, t1 = timed(False, args.steps, args.warmup, True)
    clocks = sampler.stop(t0, t1)
    k_ms = statistics.mean(a.elapsed_time(b) for a, b in kernel_events)
    k_ms_t = torch.tensor([k_ms], device=device)
    if world > 1:
        dist.all_reduce(k_ms_t, op=dist.ReduceOp.MAX)
    k_ms = k_ms_t.item()
    ms_e2e, _, _ = timed(True, args.steps, args.warmup, False)

    if rank == 0:
        peak, how = measured_peaks()
        alg = meta["alg_bytes_rank"]
        achieved = alg / (k_ms * 1e-3) / 1e9
        line = {"metric": "decode tokens/s", "value": args.batch / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "clocks": clocks,
                "e2e": {"value": args.batch / (ms_e2e * 1e-3), "unit": "tok/s",
                        "h2d_bytes_per_step": int(x_host.numel()), "d2h_bytes_per_step": int(y_host.numel())},
                "gpu_launches": args.steps * (grp.launches_per_run or len(weights)),
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "frac_of_8TBs": achieved / HBM_NOMINAL_GBS,
                             "traffic": int(alg * DRAM_TRAFFIC_RATIO[fmt]) if args.batch <= 8 else None,
                             "peak_source": f"{how} copy bandwidth",
                             "kernel": "gemv_grouped_kernel" if args.batch <= 8 else "gemm_e2m1_tc_kernel (one call per matrix)",
                             "kernel_ms": k_ms, "algorithmic_bytes_per_launch": alg},
                "pack_seconds": meta["pack_seconds"], "exchange": exchange}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_reference_leg(args.workload, args.batch, args.cpu_budget)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
