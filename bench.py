#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Default workload (`nvfp4_quantize`): NVFP4 dynamic block quantize of a bf16 [8192, 8192]
tensor ~ N(0,1) with 1 % of the elements scaled x50 (seed 1): packed E2M1 codes plus E4M3
block scales in the swizzled 128x4 layout and the fp32 global scale.  A step is one pass of
the quantize kernel over one such tensor per GPU; with N GPUs every rank quantizes its own
tensor (rows shard freely, no collective), so scaling is weak.  `value` is the algorithmic
bytes (2.5625 B per element: bf16 in, 4-bit code and 1/16 scale byte out) of all ranks per
second with inputs resident in HBM; `e2e` is the same metric through the public API with
host buffers (pinned host -> device copy, abs-max, quantize, device -> host copy of codes
and scales inside the timed region).

One JSON line is printed by rank 0.  `--impl reference` times the CPU restatement of the
reference's eager semantics (oracle/) on the host cores for the same metric.
Other workloads (`--workload fp8_gemm|nvfp4_gemm|fp8_quantize|nvfp4_stack|tp_stack`) print the same kind of line
for the GEMM sweep, the per-token FP8 quantize and the decoder linear stacks.
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
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS = COLS = 8192
ALG_BYTES_PER_ELEM = 2 + 0.5 + 1.0 / 16  # bf16 read, packed code write, block-scale write
L2_ROTATION = 4                           # distinct input tensors cycled through (4 x 134 MB > 126 MB L2)


# ----------------------------------------------------------------------------- helpers
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_input(seed: int, rows: int = ROWS, cols: int = COLS) -> torch.Tensor:
    """bf16 [rows, cols] ~ N(0,1), 1 % of the elements x50; generated on the CPU so the oracle
    and the device see identical bits."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x[torch.rand(rows, cols, generator=g) < 0.01] *= 50
    return x.bfloat16()


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist

    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed(fn, steps, warmup, world):
    """W warm-up calls, then exactly `steps` calls between CUDA events on the current stream,
    bracketed by barrier + synchronize; returns max-over-ranks milliseconds for all steps."""
    for i in range(warmup):
        fn(i)
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


# ----------------------------------------------------------------------------- CPU baseline (oracle)
def cpu_nvfp4_quantize_sample(budget_rows: int = ROWS, repeats: int = 7):
    """Times the oracle's NVFP4 quantize on a [budget_rows, 8192] slab of the workload with
    every host thread torch can use; returns (GB/s, cores, description)."""
    import oracle as o

    torch.set_num_threads(os.cpu_count() or 1)
    x = make_input(1, budget_rows, COLS)
    amax = x.float().abs().max()
    o.nvfp4_quantize(x[:64], amax)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        p, s, g = o.nvfp4_quantize(x, amax)
        o.swizzle_scales(s)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    gbs = budget_rows * COLS * ALG_BYTES_PER_ELEM / t / 1e9
    return gbs, torch.get_num_threads(), f"[{budget_rows}, {COLS}] bf16 slab of the workload, median of {repeats} passes, {t:.2f} s each"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = ROWS  # a "step" is one pass over the whole tensor (under a second on 8 cores)
    import oracle as o

    torch.set_num_threads(os.cpu_count() or 1)
    x = make_input(1, rows, COLS)
    amax = x.float().abs().max()
    for _ in range(max(1, min(args.warmup, 1))):
        o.nvfp4_quantize(x[:128], amax)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        p, s, g = o.nvfp4_quantize(x, amax)
        o.swizzle_scales(s)
    dt = time.perf_counter() - t0
    gbs = rows * COLS * ALG_BYTES_PER_ELEM * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": "nvfp4_quantize_throughput", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "nvfp4_quantize bf16 [8192, 8192], N(0,1) with 1% x50 outliers, seed 1"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"[{rows}, {COLS}] (the full tensor) per step; CPU restatement of the reference's eager semantics "
                                   "(the reference's own implementation lives in packages absent from this image)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- extras (GEMM sweep etc.)
def gemm_extras(capi, peaks, quick=True):
    """Short device-timed sweep of the quantized GEMMs: TFLOP/s per shape (rank 0, N = 1)."""
    out = {}
    shapes = [(2048, 4096, 4096), (8192, 8192, 8192)] if quick else \
        [(m, n, k) for m in (1, 16, 128, 2048, 8192) for (n, k) in ((4096, 4096), (14336, 4096), (4096, 14336), (8192, 8192))]
    for kind in ("fp8", "nvfp4"):
        res = {}
        for (M, N, K) in shapes:
            try:
                g = torch.Generator(device="cuda").manual_seed(2)
                x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=g)
                w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, generator=g) * 0.02
                bias = (torch.randn(N, device="cuda", generator=g) * 0.01).bfloat16()
                if kind == "fp8":
                    xa = capi.fp8_quantize(x, None)
                    wa = capi.fp8_quantize(w, capi.row_amax(w))
                    fn = lambda: capi.fp8_gemm(xa[0], xa[1], wa[0], wa[1], bias)  # noqa: E731
                else:
                    xa = capi.nvfp4_quantize(x, capi.amax(x))
                    wa = capi.nvfp4_quantize(w, capi.amax(w))
                    fn = lambda: capi.nvfp4_gemm(xa[0], xa[1], xa[2], wa[0], wa[1], wa[2], bias)  # noqa: E731
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                iters = 10
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / iters
                if capi.device_status() != 0:
                    res[f"{M}x{N}x{K}"] = {"error": "device-side wait timed out"}
                    continue
                res[f"{M}x{N}x{K}"] = {"ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1)}
            except Exception as exc:  # keep the headline line even if an extra fails
                res[f"{M}x{N}x{K}"] = {"error": str(exc)[:200]}
        out[kind + "_gemm"] = res
    return out


def quantize_extras(capi):
    """Device-timed GB/s of the other memory-bound kernels on inputs larger than L2."""
    out = {}

    def time_it(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    for rows, cols in ((16384, 4096), (8192, 8192), (16384, 14336)):
        xs = [torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
        n = rows * cols
        ms = time_it(lambda i=0: capi.fp8_quantize(xs[i % 3], None))
        out[f"fp8_per_token_quantize_{rows}x{cols}"] = {"ms": round(ms, 4), "GBps": round((3 * n + 4 * rows) / ms / 1e6, 1)}
        ms = time_it(lambda i=0: capi.amax(xs[i % 3]))
        out[f"amax_{rows}x{cols}"] = {"ms": round(ms, 4), "GBps": round(2 * n / ms / 1e6, 1)}
        am = capi.amax(xs[0])
        ms = time_it(lambda i=0: capi.nvfp4_quantize(xs[i % 3], am))
        out[f"nvfp4_quantize_{rows}x{cols}"] = {"ms": round(ms, 4), "GBps": round(ALG_BYTES_PER_ELEM * n / ms / 1e6, 1)}
        del xs
    return out


# ----------------------------------------------------------------------------- main arm
def run_b200(args):
    rank, world, local = dist_setup(args.gpus)
    import tensorrt_b200
    from tensorrt_b200 import capi

    peaks = measured_peaks()
    dev = torch.device("cuda", local)
    hosts = [make_input(1 + i).pin_memory() for i in range(L2_ROTATION)]  # seed 1 is the named configuration
    xs = [h.to(dev, non_blocking=True) for h in hosts]
    amaxes = [capi.amax(x) for x in xs]
    codes = torch.empty(ROWS, COLS // 2, dtype=torch.uint8, device=dev)
    sf = torch.empty(capi.nvfp4_scale_bytes(ROWS, COLS), dtype=torch.uint8, device=dev)
    gs = torch.empty((), dtype=torch.float32, device=dev)
    lib = tensorrt_b200.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()

    def step(i):
        j = i % L2_ROTATION
        rc = lib.b200q_nvfp4_quantize(xs[j].data_ptr(), 2, ROWS, COLS, amaxes[j].data_ptr(), codes.data_ptr(),
                                      sf.data_ptr(), gs.data_ptr(), stream)
        if rc != 0:
            raise RuntimeError(f"b200q_nvfp4_quantize returned {rc}")

    with ClockSampler(local) as clocks:
        ms = timed(step, args.steps, args.warmup, world)
    alg_bytes = ROWS * COLS * ALG_BYTES_PER_ELEM
    value = alg_bytes * world * args.steps / (ms * 1e-3) / 1e9
    kernel_ms = ms / args.steps

    # end to end through the public API with host buffers
    h_codes = torch.empty(ROWS, COLS // 2, dtype=torch.uint8).pin_memory()
    h_sf = torch.empty(sf.numel(), dtype=torch.uint8).pin_memory()

    def e2e_step(i):
        x = hosts[i % L2_ROTATION].to(dev, non_blocking=True)
        c, s, g = capi.nvfp4_quantize(x, capi.amax(x))
        h_codes.copy_(c, non_blocking=True)
        h_sf.copy_(s, non_blocking=True)
        g.item()  # device -> host read of the result's global scale: completes the step

    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = timed(e2e_step, e2e_steps, 2, world)
    e2e_value = alg_bytes * world * e2e_steps / (e2e_ms * 1e-3) / 1e9

    line = {
        "metric": "nvfp4_quantize_throughput", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "nvfp4_quantize bf16 [8192, 8192] per GPU, N(0,1) with 1% x50 outliers, seed 1; "
                               "codes + swizzled E4M3 block scales + fp32 global scale; amax supplied as op input",
                   "l2": f"inputs rotate over {L2_ROTATION} distinct 134 MB tensors (> 126 MB L2)",
                   "sharding": "one tensor per rank, no collective"},
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": ROWS * COLS * 2,
                "d2h_bytes_per_step": int(codes.numel() + sf.numel() + 4), "steps": e2e_steps,
                "ms_per_step": e2e_ms / e2e_steps,
                "path": "pinned host bf16 -> device, b200q_amax + b200q_nvfp4_quantize, codes/scales -> pinned host"},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": alg_bytes / (kernel_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": alg_bytes / (kernel_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "peak_source": f"{peaks['source']} HBM copy bandwidth", "traffic": NCU_TRAFFIC_BYTES,
                     "kernel": "nvfp4_quantize_kernel<bf16, codes>", "algorithmic_bytes_per_launch": alg_bytes},
    }
    if rank == 0 and world == 1:
        gbs, cores, sample = cpu_nvfp4_quantize_sample()
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
        if not args.no_extras:
            line["extras"] = gemm_extras(capi, peaks)
            line["extras"]["quantize"] = quantize_extras(capi)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


# DRAM bytes (read + write) per launch of the quantize kernel on this workload, from the
# committed ncu capture (profiles/nvfp4_quantize_kernel_bf16_8192x8192.md).
NCU_TRAFFIC_BYTES = 155_108_352


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="nvfp4_quantize")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--shape", default="", help="M,N,K for the GEMM workloads (default: the whole sweep)")
    ap.add_argument("--micro-batches", type=int, default=0, dest="micro_batches",
                    help="tp_stack: micro-batches of tokens walking the layers on separate streams (exchange / GEMM overlap); "
                         "0 = 4, or 8 at TP >= 8")
    ap.add_argument("--fused", type=int, default=1, help="tp_stack: 1 = fused GEMM + peer-memory all-reduce, 0 = NCCL")
    ap.add_argument("--decode-graph", type=int, default=-1, dest="decode_graph",
                    help="tp_stack: 1 = replay the decode step as a CUDA graph, 0 = issue it launch by launch, "
                         "-1 = graph on one GPU only")
    ap.add_argument("--phase", choices=["all", "prefill", "decode"], default="all",
                    help="tp_stack: time only the prefill or only the decode step (profiling runs)")
    ap.add_argument("--layers", type=int, default=0, help="tp_stack / nvfp4_stack: override the layer count (profiling runs; 0 = the config's)")
    ap.add_argument("--sharded", type=int, default=1,
                    help="tp_stack prefill: 1 = token-sharded residual stream (reduce-scatter + all-gather of FP8 codes), "
                         "0 = all-reduce")
    ap.add_argument("--slabs", type=int, default=1, help="row slabs per row-parallel linear (all-reduce overlap) in tp_stack")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload != "nvfp4_quantize":
        from tensorrt_b200 import bench_workloads

        bench_workloads.run(args)
        return
    run_b200(args)


if __name__ == "__main__":
    main()
