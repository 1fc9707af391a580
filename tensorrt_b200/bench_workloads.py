"""Secondary benchmark workloads of `bench.py --workload NAME` (one JSON line each).

fp8_gemm / nvfp4_gemm   quantized-linear GEMM sweep: M in {1, 16, 128, 2048, 8192} x
                        (N, K) in {(4096, 4096), (14336, 4096), (4096, 14336), (8192, 8192)},
                        x ~ N(0,1) bf16, W ~ N(0, 0.02) bf16, bias ~ N(0, 0.01); `--shape M,N,K`
                        restricts the sweep to one shape.  value = TFLOP/s of the largest
                        shape; every shape is listed under "shapes" with its roofline
                        fraction (tensor peak for M >= 2048, HBM for M <= 128).
fp8_quantize            per-token FP8 quantize of bf16 [16384, 4096]; value = GB/s.
nvfp4_stack             NVFP4 W4A4 decoder linear stack (hidden 4096, 32 q / 8 kv heads of 128,
                        FFN 14336, 32 layers), prefill of 8 x 2048 tokens; value = tokens/s.
tp_stack                FP8 tensor-parallel decoder linear stack (hidden 8192, 64 q / 8 kv heads,
                        FFN 28672, 80 layers) at TP = --gpus; value = prefill tokens/s, decode
                        tokens/s reported beside it.
"""
from __future__ import annotations

import json
import os

import torch

SWEEP_M = (1, 16, 128, 2048, 8192)
SWEEP_NK = ((4096, 4096), (14336, 4096), (4096, 14336), (8192, 8192))


def _peaks():
    import bench

    return bench.measured_peaks()


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def gemm_case(capi, kind, M, N, K, seed, iters):
    g = torch.Generator(device="cuda").manual_seed(seed)
    # several operand sets so that consecutive iterations do not find their operands in L2
    # when they are small enough to fit there
    nsets = max(1, min(8, int(300e6 // max(1, (M + N) * K))))
    sets = []
    for _ in range(nsets):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, generator=g)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, generator=g) * 0.02
        bias = (torch.randn(N, device="cuda", generator=g) * 0.01).bfloat16()
        if kind == "fp8":
            sets.append((capi.fp8_quantize(x, None), capi.fp8_quantize(w, capi.row_amax(w)), bias))
        else:
            sets.append((capi.nvfp4_quantize(x, capi.amax(x)), capi.nvfp4_quantize(w, capi.amax(w)), bias))
        del x, w
    it = [0]

    def fn():
        xa, wa, bias = sets[it[0] % nsets]
        it[0] += 1
        if kind == "fp8":
            capi.fp8_gemm(xa[0], xa[1], wa[0], wa[1], bias)
        else:
            capi.nvfp4_gemm(xa[0], xa[1], xa[2], wa[0], wa[1], wa[2], bias)

    if M <= 128:
        # decode-sized calls are shorter than the host work of issuing them: time them the way a
        # serving loop runs them, as a CUDA graph of back-to-back launches over the operand sets,
        # with the weights declared static (quantized and complete long before the launches)
        torch.cuda.synchronize()
        capi.assume_static_weights(True)
        reps = max(nsets, 16)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(reps):
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        capi.assume_static_weights(False)
        ms = _time(graph.replay, iters) / reps
    else:
        ms = _time(fn, iters)
    if capi.device_status() != 0:
        raise RuntimeError("device-side wait timed out")
    return ms


def run_gemm(args, kind):
    import bench
    from tensorrt_b200 import capi

    torch.cuda.set_device(0)
    peaks = _peaks()
    scale = 2.0 if kind == "fp8" else 4.0
    tensor_peak = peaks["bf16_tflops"] * scale          # measured bf16 burst x2 (FP8) / x4 (FP4)
    nominal = 4500.0 if kind == "fp8" else 9000.0
    bytes_per_elem = 1.0 if kind == "fp8" else 0.5 + 1.0 / 16
    if args.shape:
        shapes = [tuple(int(v) for v in args.shape.split(","))]
    else:
        shapes = [(m, n, k) for (n, k) in SWEEP_NK for m in SWEEP_M]
    results = {}
    with bench.ClockSampler(0) as clocks:
        for idx, (M, N, K) in enumerate(shapes):
            ms = gemm_case(capi, kind, M, N, K, seed=2 + idx, iters=max(5, args.steps))
            flops = 2.0 * M * N * K
            byts = (M + N) * K * bytes_per_elem + 2.0 * M * N + (4 * (M + N) if kind == "fp8" else 0) + 2 * N
            tf = flops / ms / 1e9
            gbs = byts / ms / 1e6
            entry = {"ms": round(ms, 5), "tflops": round(tf, 1), "GBps": round(gbs, 1)}
            if M >= 2048:
                entry["bound"] = "tensor"
                entry["frac_of_measured_scaled_peak"] = round(tf / tensor_peak, 3)
                entry["frac_of_nominal_dense_peak"] = round(tf / nominal, 3)
            else:
                entry["bound"] = "hbm"
                entry["frac_of_measured_hbm"] = round(gbs / peaks["hbm_gbs"], 3)
            results[f"{M}x{N}x{K}"] = entry
    M, N, K = shapes[-1]
    head = results[f"{M}x{N}x{K}"]
    line = {
        "metric": f"{kind}_quant_linear_gemm_throughput", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": 3, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "e4m3xe4m3->f32" if kind == "fp8" else "e2m1xe2m1(ue4m3 block scales)->f32",
        "data": "synthetic",
        "config": {"workload": f"{kind} quantized-linear GEMM sweep, headline shape M,N,K = {M},{N},{K}; x ~ N(0,1), "
                               "W ~ N(0,0.02), bias ~ N(0,0.01); operands pre-quantized and resident in HBM",
                   "l2": "operand sets rotate so that sets smaller than L2 are not re-read from L2",
                   "small_m": "M <= 128: timed as a CUDA graph of back-to-back launches (host issue time excluded), "
                              "weights declared static (b200q_gemm_assume_static_weights)"},
        "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "achieved": head["tflops"], "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": head["tflops"] / tensor_peak,
                     "peak_source": f"{peaks['source']} cuBLAS bf16 burst x{int(scale)}; nominal dense {nominal:.0f}",
                     "traffic": None},
        "shapes": results,
    }
    print(json.dumps(line))


def run_fp8_quantize(args):
    import bench
    from tensorrt_b200 import capi

    torch.cuda.set_device(0)
    peaks = _peaks()
    rows, cols = 16384, 4096
    xs = [torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    it = [0]

    def fn():
        capi.fp8_quantize(xs[it[0] % 3], None)
        it[0] += 1

    with bench.ClockSampler(0) as clocks:
        ms = _time(fn, max(10, args.steps))
    byts = 3.0 * rows * cols + 4.0 * rows
    gbs = byts / ms / 1e6
    print(json.dumps({
        "metric": "fp8_per_token_quantize_throughput", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": f"per-token FP8 E4M3 quantize of bf16 [{rows}, {cols}] ~ N(0,1), row abs-max reduced in the kernel",
                                        "l2": "3 rotating inputs of 134 MB"},
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "peak_source": f"{peaks['source']} HBM copy bandwidth", "traffic": None}}))


def run(args):
    if args.workload == "fp8_gemm":
        run_gemm(args, "fp8")
    elif args.workload == "nvfp4_gemm":
        run_gemm(args, "nvfp4")
    elif args.workload == "fp8_quantize":
        run_fp8_quantize(args)
    elif args.workload in ("nvfp4_stack", "tp_stack"):
        from . import stack_bench

        stack_bench.run(args)
    else:
        raise SystemExit(f"unknown workload {args.workload!r}")
