#!/usr/bin/env python
"""Benchmark of the fused 4-bit dequant-GEMV path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode7b|decode7b_e2m1|decode70b|e2m1_4096|gf4_11008] [--batch B]

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
epilogue plus a barrier (--exchange fused) or by one NCCL all-gather per step
(--exchange nccl); the default, auto, takes fused when symmetric memory is
available and says which one ran.

Rank 0 prints one JSON line: metric, value, unit, per-step time, clocks seen
during the timed region, the end-to-end figure with host copies (e2e), the
roofline of the dominant kernel, a parity record (device results against the
CPU oracle, computed outside the timed region) and (N = 1) a CPU baseline.
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

import numpy as np  # noqa: E402
import torch  # noqa: E402

HBM_NOMINAL_GBS = 8000.0
PARITY_GATE = 1e-3
# DRAM bytes (read + write) per algorithmic byte of each dominant kernel, from one ncu capture each on a smaller
# case of the same kernel (16 x 11008 x 4096 GF4 at batch 1 and at batch 16, 16 x 8192 x 8192 E2M1 at batch 16 and
# at batch 1); traffic grows in proportion to the rows processed, so a full launch's traffic is this ratio times its
# algorithmic bytes.
DRAM_TRAFFIC_RATIO = {
    "gf4_lut2_kernel": (377.961216 + 5.431552) / 378.101760,
    "gemm_ta_kernel<gf4>": (380.471808 + 8.067328) / 385.351680,
    "gemm_ta_kernel<e2m1>": (621.232640 + 6.949376) / 612.368384,
    "gemv_grouped_kernel": 608.581888 / 604.504064,      # E2M1; GF4 reaches this kernel only for ungrouped or short rows
}

WORKLOADS = {
    # name: (fmt, group, had_block, layers, [(label, N, K, count-per-layer)], init std, seed)
    "decode7b": ("gf4", 128, 128, 32, [("qkvo", 4096, 4096, 4), ("gate_up", 11008, 4096, 2), ("down", 4096, 11008, 1)], 0.02, 3),
    "decode7b_e2m1": ("e2m1", 32, 0, 32, [("qkvo", 4096, 4096, 4), ("gate_up", 11008, 4096, 2), ("down", 4096, 11008, 1)], 0.02, 6),
    "decode70b": ("e2m1", 32, 0, 80, [("qo", 8192, 8192, 2), ("kv", 1024, 8192, 2), ("gate_up", 28672, 8192, 2),
                                       ("down", 8192, 28672, 1)], 0.015, 4),
    "e2m1_4096": ("e2m1", 32, 0, 16, [("linear", 4096, 4096, 1)], 0.02, 1),
    # the 70B-class attention projection alone: the batched kernel's sweep shape (16, 32, 64 rows)
    "e2m1_8192": ("e2m1", 32, 0, 16, [("linear", 8192, 8192, 1)], 0.02, 5),
    "gf4_11008": ("gf4", 128, 128, 16, [("linear", 11008, 4096, 1)], 0.02, 2),
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
    fmt, g, had, layers, mats, std, seed = WORKLOADS[name]
    spec = jq.QuantSpec(fmt, g, had)
    gen = torch.Generator("cpu").manual_seed(seed)
    proto, head_rows = {}, {}
    t0 = time.time()
    for label, N, K, _ in mats:
        if N % world:
            raise SystemExit(f"N={N} of {label} does not divide over {world} ranks")
        lo, hi = rank * (N // world), (rank + 1) * (N // world)
        W = torch.randn(N, K, generator=gen) * std     # every rank draws the same matrix, keeps its rows
        if fmt == "e2m1":
            W = W.bfloat16().float()
        head_rows[label] = W[lo:lo + 2].clone()        # two source rows for the packer check against the oracle
        proto[label] = jq.pack_weight(W[lo:hi].to(device), spec, threads=threads)   # quantised on the GPU
        del W
    pack_s = time.time() - t0
    weights, labels = [], []
    for _layer in range(layers):
        for label, N, K, cnt in mats:
            for _ in range(cnt):
                p = proto[label]
                weights.append(jq.PackedWeight(p.spec, p.N, p.K, p.qweight.clone(),
                                               None if p.scales is None else p.scales.clone(),
                                               None if p.codebook is None else p.codebook.clone()))
                labels.append(label)
    alg = sum(jq.algorithmic_bytes(spec, w.N, w.K, batch, 2, 2) for w in weights)
    meta = {"spec": spec, "pack_seconds": pack_s, "alg_bytes_rank": alg, "n_matrices": len(weights),
            "weights_total": sum(w.N * w.K for w in weights), "proto": proto, "head_rows": head_rows,
            "labels": labels}
    return weights, meta


# ---- parity against the CPU oracle (outside the timed region) ---------------------------------------------------
def oracle_dequant(pw):
    from oracle import formats
    codes = formats.unpack_nibbles(pw.qweight.cpu().numpy(), pw.K)
    s = None if pw.scales is None else pw.scales.cpu().numpy()
    if pw.spec.fmt == "e2m1":
        return formats.dequant_e2m1(codes, s, pw.spec.group_size)
    return formats.dequant_gf4(codes, pw.codebook.cpu().numpy(), s, pw.spec.group_size)


def parity_record(meta, grp, batch, device):
    """One matrix per distinct shape: device dequantisation and the packer's
    first rows bit for bit against the oracle, and the outputs the timed
    launch produced against the oracle's fp32 reference on the same inputs."""
    from if_i_could_turn_back_time_b200 import ops
    from oracle import formats, jenks
    spec = meta["spec"]
    seen, rec = set(), {"dequant_bit_exact": True, "codes_bit_exact": True, "timed_outputs_bit_exact": True, "timed_outputs_rel_err_bf16": 0.0, "max_rel_err": 0.0,
                        "gate": PARITY_GATE, "matrices_checked": 0}
    for i, label in enumerate(meta["labels"]):
        if label in seen:
            continue
        seen.add(label)
        pw = grp.weights[i]
        w_hat = oracle_dequant(pw)
        rec["dequant_bit_exact"] &= bool(np.array_equal(ops.dequantize(pw).cpu().numpy(), w_hat))
        rows = meta["head_rows"][label].numpy()
        if spec.had_block:
            rows = formats.fwht_block(rows, spec.had_block)
        if spec.fmt == "e2m1":
            c, _ = formats.quantize_e2m1(rows, spec.group_size)
        else:
            c, _, _ = jenks.quantize_gf4(rows, spec.group_size)
        rec["codes_bit_exact"] &= bool(np.array_equal(formats.pack_nibbles(c), pw.qweight[:2].cpu().numpy()))
        # the same kernel family with fp32 outputs against the fp32 oracle (a bf16 output cannot itself meet
        # 1e-3: half a bf16 ulp is 2e-3), and the timed launch's bf16 outputs against that result rounded to bf16
        x = grp.xs[i]
        lo = grp.row_offsets[i]
        y32 = ops.linear(x, pw, out_dtype=torch.float32)
        ref = formats.linear_ref(x.float().cpu().numpy(), w_hat, None, had_block=spec.had_block)
        rec["max_rel_err"] = max(rec["max_rel_err"], float(formats.rel_err(y32.cpu().numpy(), ref)))
        yt = grp.ys[i][:, lo:lo + pw.N]
        rec["timed_outputs_bit_exact"] &= bool(torch.equal(yt, y32.to(yt.dtype)))   # (false where a grouped launch and a
        #                                   single call pick different kernels or K tilings: summation order only)
        rec["timed_outputs_rel_err_bf16"] = max(rec["timed_outputs_rel_err_bf16"],
                                                float(formats.rel_err(yt.float().cpu().numpy(), ref)))
        rec["matrices_checked"] += 1
    # gate on the fp32 outputs; the timed bf16 outputs may add one bf16 rounding step (2^-8 of the largest output)
    rec["pass"] = bool(rec["dequant_bit_exact"] and rec["codes_bit_exact"] and rec["max_rel_err"] <= PARITY_GATE
                       and rec["timed_outputs_rel_err_bf16"] <= 2.0 ** -8 + PARITY_GATE)
    return rec


# ---- the reference's forward form on the host cores ----------------------------------------------------------------
def cpu_layerset(name: str, batch: int, frac: float = 1.0):
    """Random packed tensors with the shapes of one layer set (row fraction
    frac of every matrix) and a closure running the reference's per-call form
    over them: unpack -> table lookup -> times the group scale -> fp32 F.linear
    (Python_Jenks_Test/Jenks_Tests/Quantization_Experiments/layers.py:36-38).
    Timing depends on shapes and dtypes only, so codes, codebooks and scales
    are seeded random values; nothing of the CUDA library is involved."""
    from oracle import ref_linear
    fmt, g, had, layers, mats, std, seed = WORKLOADS[name]
    gen = torch.Generator("cpu").manual_seed(1000 + seed)
    items = []
    for label, N, K, cnt in mats:
        rows = max(1, int(round(N * frac)))
        q = torch.randint(0, 256, (rows, K // 2), generator=gen, dtype=torch.uint8)
        s = (torch.rand(rows, K // g, generator=gen) * 0.05 + 0.01).half()
        cb = torch.sort(torch.randn(rows, 16, generator=gen), dim=1).values.half() if fmt == "gf4" else None
        x = torch.randn(batch, K, generator=gen).bfloat16()
        items.append((cnt, rows, K, q, s, cb, x))

    def run():
        for cnt, rows, K, q, s, cb, x in items:
            for _ in range(cnt):
                ref_linear.per_call(x, q, s, cb, None, rows, K, g, had)

    weights_set = sum(n * k * c for _, n, k, c in mats)
    return run, layers, weights_set


def cpu_baseline_leg(name: str, batch: int, budget_s: float):
    """One full layer set per pass, as many passes as fit the budget (at least
    3), median; tokens/s = batch / (pass time x layers)."""
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    run, layers, wset = cpu_layerset(name, batch, 1.0)
    run()
    t = time.perf_counter(); run(); one = time.perf_counter() - t
    reps = max(3, min(30, int(budget_s / max(one, 1e-3))))
    times = []
    for _ in range(reps):
        t = time.perf_counter(); run(); times.append(time.perf_counter() - t)
    med = statistics.median(times)
    fmt, g, had = WORKLOADS[name][:3]
    return {"value": batch / (med * layers), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"one full layer set ({wset / 1e6:.0f} M weights, {fmt} g{g}), {reps} passes, median {med * 1e3:.0f} ms; "
                      f"per-call dequantise + fp32 F.linear in PyTorch on CPU; x {layers} layers per token"}


def reference_arm(args, config):
    """--impl reference: the same CPU form, each step a bounded sample (a row
    fraction of every matrix of one layer set, the whole set when it fits the
    per-step budget); ms_per_step is the measured time of that sample."""
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    run, layers, wset = cpu_layerset(args.workload, args.batch, 1.0)
    run()
    t = time.perf_counter(); run(); full = time.perf_counter() - t
    steps_total = args.steps + max(args.warmup, 1)
    frac = min(1.0, (150.0 / steps_total) / max(full, 1e-3))      # the whole run stays within a few minutes
    if frac < 1.0:
        frac = max(frac, 1.0 / 512)
        run, layers, wset = cpu_layerset(args.workload, args.batch, frac)
        run()
    for _ in range(max(args.warmup, 1)):
        run()
    times = []
    for _ in range(args.steps):
        t = time.perf_counter(); run(); times.append(time.perf_counter() - t)
    step_s = statistics.mean(times)
    tok_s = args.batch / (step_s / frac * layers)
    cb = {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port",
          "sample": f"row fraction {frac:.4f} of every matrix of one layer set per step ({wset * frac / 1e6:.1f} M weights); "
                    f"per-call dequantise + fp32 F.linear in PyTorch on CPU; tokens/s = batch / (step time / fraction x {layers} layers)"}
    return {"impl": "reference", "metric": "decode tokens/s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": cb,
            "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


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
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: all-gather fused into the GEMV epilogue (peer stores) or one NCCL all-gather per step; "
                         "auto = fused where symmetric memory is available, else nccl; an explicit choice fails loudly")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    fmt, g, had, layers, mats, std, _seed = WORKLOADS[args.workload]
    config = {"workload": f"{args.workload}: {layers} layers x " + ", ".join(f"{c}x{n}x{k}" for _, n, k, c in mats) +
                          f", {fmt} g{g}" + (f" + block-Hadamard-{had}" if had else "") + f", batch {args.batch}, bf16 activations",
              "batch": args.batch, "parallelism": f"row-shard x{world} + all-gather" if world > 1 else "single GPU",
              "l2": "inputs larger than L2 (every matrix has its own allocation; one step streams them all once)"}

    if args.impl == "reference":
        if rank != 0:
            return
        print(json.dumps(reference_arm(args, config)))
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

    def make_group(fused: bool):
        if fused:
            return ops.GroupedGemv(weights, args.batch, torch.bfloat16, full_rows=[w.N * world for w in weights],
                                   row_offsets=[w.N * rank for w in weights], group=dist.group.WORLD)
        return ops.GroupedGemv(weights, args.batch, torch.bfloat16)

    exchange, want_fused = "none", False
    if world > 1:
        want_fused = args.exchange in ("auto", "fused")
    grps = None
    if want_fused:
        try:
            grps = [make_group(True), make_group(True)]   # two sets of arenas: the end-to-end loop uploads one while the other runs
            if not grps[0].fused_exchange:
                raise RuntimeError("this batch has no kernel with the fused epilogue")
            exchange = "fused peer stores + barrier"
        except Exception as e:
            if args.exchange == "fused":
                raise SystemExit(f"--exchange fused was requested but is unavailable: {type(e).__name__}: {e}")
            if rank == 0:
                print(f"fused exchange unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
            grps = None
    if grps is None:
        grps = [make_group(False), make_group(False)]
        if world > 1:
            exchange = "nccl all_gather_into_tensor"
    fused = grps[0].fused_exchange
    grp = grps[0]
    gen = torch.Generator("cpu").manual_seed(100)
    x_host = torch.empty(grp.x_arena.numel(), dtype=torch.uint8).pin_memory()
    x_host.view(torch.bfloat16).copy_(torch.randn(grp.x_arena.numel() // 2, generator=gen).bfloat16())
    y_bytes = grp.y_arena.numel() * (1 if fused else world)
    y_host = torch.empty(y_bytes, dtype=torch.uint8).pin_memory()
    for gobj in grps:
        gobj.x_arena.copy_(x_host)
    y_all = [torch.empty(y_bytes, dtype=torch.uint8, device=device) if (world > 1 and not fused) else None for _ in grps]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    kernel_events = []

    def device_step(i: int, record: bool = False):
        gobj = grps[i & 1]
        if record:
            a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
            a.record()
        gobj.run()
        if record:
            b.record()
            kernel_events.append((a, b))
        if fused:
            gobj.barrier()
        elif world > 1:
            dist.all_gather_into_tensor(y_all[i & 1], gobj.y_arena)

    def timed_device(steps: int, warmup: int):
        for i in range(warmup):
            device_step(i)
        barrier()
        t0 = time.time()
        start = torch.cuda.Event(enable_timing=True); end = torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            device_step(i, True)
        end.record()
        barrier()
        t1 = time.time()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps, t0, t1

    # End to end through the public API with host buffers: every step uploads that step's activations from pinned
    # memory and (rank 0, which owns the result) reads the gathered outputs back.  Two sets of arenas alternate, so
    # the copy engine uploads step i + 1 and downloads step i - 1 while step i computes; every copy of every step
    # is inside the timed region.
    copy_stream = torch.cuda.Stream(device=device)
    main_stream = torch.cuda.current_stream(device)

    def timed_e2e(steps: int, warmup: int):
        up_done = [torch.cuda.Event(), torch.cuda.Event()]
        run_done = [torch.cuda.Event(), torch.cuda.Event()]
        down_done = [torch.cuda.Event(), torch.cuda.Event()]

        def upload(i):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(run_done[i & 1])          # the step that last read this arena is over
                grps[i & 1].x_arena.copy_(x_host, non_blocking=True)
                up_done[i & 1].record(copy_stream)

        def loop(n):
            upload(0)
            for i in range(n):
                if i + 1 < n:
                    upload(i + 1)
                main_stream.wait_event(up_done[i & 1])
                main_stream.wait_event(down_done[i & 1])        # the download of step i - 2 has left this arena
                device_step(i)
                run_done[i & 1].record(main_stream)
                if rank == 0:
                    with torch.cuda.stream(copy_stream):
                        copy_stream.wait_event(run_done[i & 1])
                        src = y_all[i & 1] if y_all[i & 1] is not None else grps[i & 1].y_arena
                        y_host.copy_(src, non_blocking=True)
                        down_done[i & 1].record(copy_stream)
            copy_stream.synchronize()
            main_stream.synchronize()

        for ev in run_done + down_done:
            ev.record(main_stream)
        loop(max(warmup, 2))
        barrier()
        start = torch.cuda.Event(enable_timing=True); end = torch.cuda.Event(enable_timing=True)
        start.record(main_stream)
        loop(steps)
        for ev in down_done:
            main_stream.wait_event(ev)                          # the last downloads are inside the timed region
        end.record(main_stream)
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    ms_step, t0, t1 = timed_device(args.steps, args.warmup)
    clocks = sampler.stop(t0, t1)
    k_ms = statistics.mean(a.elapsed_time(b) for a, b in kernel_events)
    k_ms_t = torch.tensor([k_ms], device=device)
    if world > 1:
        dist.all_reduce(k_ms_t, op=dist.ReduceOp.MAX)
    k_ms = k_ms_t.item()
    ms_e2e = timed_e2e(args.steps, args.warmup)

    # ---- parity: this rank's columns against the oracle; N > 1: every rank holds the same gathered outputs and
    #      rank 0 checks one whole (unsharded) matrix assembled from the ranks' oracle slices
    parity = None
    if not args.no_parity:
        device_step(0)
        barrier()
        status = min(gobj.status() for gobj in grps)
        parity = parity_record(meta, grps[0], args.batch, device)
        parity["device_status"] = status
        if world > 1:
            src = y_all[0] if y_all[0] is not None else grps[0].y_arena
            chk = src.view(torch.int16).to(torch.int64).sum().reshape(1)
            allchk = [torch.zeros_like(chk) for _ in range(world)]
            dist.all_gather(allchk, chk)
            parity["gathered_checksums_equal"] = bool(all(int(c) == int(allchk[0]) for c in allchk))
            if fused:
                from oracle import formats
                pw = grps[0].weights[0]
                ref = formats.linear_ref(grps[0].xs[0].float().cpu().numpy(), oracle_dequant(pw), None, had_block=meta["spec"].had_block)
                mine = torch.from_numpy(ref).to(device)
                parts = [torch.zeros_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                if rank == 0:
                    # gathered bf16 outputs of the whole matrix against the assembled fp32 oracle: within one bf16
                    # rounding step (2^-8) plus the gate
                    full = torch.cat(parts, dim=1).cpu().numpy()
                    got = grps[0].ys[0].float().cpu().numpy()
                    parity["unsharded_rel_err_bf16"] = float(formats.rel_err(got, full))
                    parity["pass"] = bool(parity["pass"] and parity["unsharded_rel_err_bf16"] <= 2.0 ** -8 + PARITY_GATE)
            parity["pass"] = bool(parity["pass"] and parity["gathered_checksums_equal"])
        parity["pass"] = bool(parity["pass"] and status == 0)

    if rank == 0:
        peak, how = measured_peaks()
        alg = meta["alg_bytes_rank"]
        achieved = alg / (k_ms * 1e-3) / 1e9
        if grp._ta:
            max_k = max(w.K for w in grp.weights)
            lut = grp.weights[0].spec.fmt == "gf4" and args.batch == 1 and max_k * 2 <= 24 * 1024
            kernel = ("gf4_lut2_kernel" if lut else "gemm_ta_kernel<%s>" % grp.weights[0].spec.fmt) + " (+ ta_prepare_kernel)"
        else:
            kernel = "gemv_grouped_kernel"
        line = {"metric": "decode tokens/s", "value": args.batch / (ms_step * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "clocks": clocks,
                "e2e": {"value": args.batch / (ms_e2e * 1e-3), "unit": "tok/s",
                        "h2d_bytes_per_step": int(x_host.numel()) * world, "d2h_bytes_per_step": int(y_host.numel()),
                        "note": "every rank uploads the step's activations; rank 0 downloads the gathered outputs; "
                                "copies of neighbouring steps overlap the kernel on a second stream"},
                "gpu_launches": args.steps * (grp.launches_per_run or len(weights)),
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "frac_of_8TBs": achieved / HBM_NOMINAL_GBS,
                             "traffic": int(alg * DRAM_TRAFFIC_RATIO[kernel.split(" ")[0]]),
                             "peak_source": f"{how} copy bandwidth", "kernel": kernel,
                             "kernel_ms": k_ms, "algorithmic_bytes_per_launch": alg},
                "parity": parity, "pack_seconds": meta["pack_seconds"], "exchange": exchange}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg(args.workload, args.batch, args.cpu_budget)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["pass"] and rank == 0:
        sys.exit(3)


if __name__ == "__main__":
    main()
