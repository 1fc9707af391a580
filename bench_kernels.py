"""Single-kernel workloads of `bench.py --workload NAME` and the `extras` of the default line.

nvfp4_quantize          NVFP4 dynamic block quantize of bf16 [8192, 8192] ~ N(0,1) with 1 % of the
                        elements x50 (seed 1): value = algorithmic GB/s (2.5625 B per element).
fp8_quantize            per-token FP8 quantize of bf16 [16384, 4096]; value = GB/s.
fp8_gemm / nvfp4_gemm   quantized-linear GEMM sweep: M in {1, 16, 128, 2048, 8192} x
                        (N, K) in {(4096, 4096), (14336, 4096), (4096, 14336), (8192, 8192)},
                        x ~ N(0,1) bf16, W ~ N(0, 0.02) bf16, bias ~ N(0, 0.01); `--shape M,N,K`
                        restricts the sweep to one shape.  value = TFLOP/s of the largest
                        shape; every shape is listed under "shapes" with its own roofline
                        object (tensor peak for M >= 2048, HBM for M <= 128).

Every number is timed with CUDA events on the launching stream over a region of at least half a
second and at least 50 launches, after warm-up, on operands that rotate through more than L2's
worth of memory.
"""
from __future__ import annotations

import json

import torch

import bench_common as bc

SWEEP_M = (1, 16, 128, 2048, 8192)
SWEEP_NK = ((4096, 4096), (14336, 4096), (4096, 14336), (8192, 8192))

# DRAM bytes (read + write) per launch of the NVFP4 quantize kernel on bf16 [8192, 8192], from an
# ncu capture of this kernel and shape (dram__bytes_read.sum + dram__bytes_write.sum).
NVFP4_QUANTIZE_NCU_TRAFFIC = 155_108_352


def time_device(fn, min_ms: float = 500.0, min_iters: int = 50, warmup: int = 3, max_iters: int = 200000):
    """ms per call of `fn()`: warm-up, then timed rounds between CUDA events until the timed region
    holds at least `min_iters` calls and lasts at least `min_ms`."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total_ms, total_n, n = 0.0, 0, min_iters
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        total_ms += e0.elapsed_time(e1)
        total_n += n
        if (total_ms >= min_ms and total_n >= min_iters) or total_n >= max_iters:
            return total_ms / total_n, total_n
        per = total_ms / total_n
        n = int(min(max_iters - total_n, max(min_iters, (min_ms - total_ms) / max(per, 1e-4) * 1.1)))


def time_graphed(fn, reps: int, min_ms: float = 500.0):
    """ms per call of `fn()` with `reps` calls captured into one CUDA graph and the graph replayed
    (time_device's rules): a launch of a few tens of microseconds issued from Python is otherwise
    timed by the host, not by the device."""
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
    ms, n = time_device(graph.replay, min_ms, min_iters=max(4, 50 // reps + 1))
    return ms / reps, n * reps


def hbm_roofline(gbs: float, peaks, alg_bytes: float, kernel: str, traffic=None):
    return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
            "peak_source": f"{peaks['source']} HBM copy bandwidth", "traffic": traffic, "kernel": kernel,
            "algorithmic_bytes_per_launch": alg_bytes}


def tensor_roofline(tflops: float, peaks, kind: str, kernel: str, flops: float):
    scale = 2.0 if kind == "fp8" else 4.0
    nominal = 4500.0 if kind == "fp8" else 9000.0
    # these launches run back to back for half a second or more, so the GPU sits at the clock its
    # power cap sustains: the sustained cuBLAS figure is the denominator, the burst one is beside it
    peak = peaks["bf16_tflops_sustained"] * scale
    return {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
            "peak_source": f"{peaks['source']} sustained cuBLAS bf16 x{int(scale)} (launches timed back to back for >= 0.5 s)",
            "frac_of_burst_scaled_peak": tflops / (peaks["bf16_tflops"] * scale), "frac_of_nominal_dense_peak": tflops / nominal,
            "traffic": None, "kernel": kernel, "algorithmic_flops_per_launch": flops}


# ----------------------------------------------------------------------------- quantize kernels
def nvfp4_quantize_case(capi, peaks, min_ms=500.0):
    """The configuration's own tensor (seed 1) plus three more of the same distribution, rotated."""
    import tensorrt_b200

    lib = tensorrt_b200.load_library()
    xs = [bc.make_input(1 + i).cuda() for i in range(bc.L2_ROTATION)]
    amaxes = [capi.amax(x) for x in xs]
    codes = torch.empty(bc.ROWS, bc.COLS // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(capi.nvfp4_scale_bytes(bc.ROWS, bc.COLS), dtype=torch.uint8, device="cuda")
    gs = torch.empty((), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    it = [0]

    def fn():
        j = it[0] % bc.L2_ROTATION
        it[0] += 1
        rc = lib.b200q_nvfp4_quantize(xs[j].data_ptr(), 2, bc.ROWS, bc.COLS, amaxes[j].data_ptr(), codes.data_ptr(), sf.data_ptr(),
                                      gs.data_ptr(), stream)
        if rc != 0:
            raise RuntimeError(f"b200q_nvfp4_quantize returned {rc}")

    ms, n = time_device(fn, min_ms)
    alg = bc.ROWS * bc.COLS * bc.ALG_BYTES_PER_ELEM
    gbs = alg / ms / 1e6
    return {"ms": ms, "launches": n, "GBps": gbs,
            "roofline": hbm_roofline(gbs, peaks, alg, "nvfp4_quantize_kernel<bf16, codes>", NVFP4_QUANTIZE_NCU_TRAFFIC)}


def quantize_suite(capi, peaks, min_ms=500.0):
    """GB/s of every memory-bound kernel of the quantize family on inputs larger than L2, each with
    its own roofline object."""
    out = {"nvfp4_quantize_8192x8192_seed1": nvfp4_quantize_case(capi, peaks, min_ms)}
    for rows, cols in ((16384, 4096), (8192, 8192), (16384, 14336)):
        xs = [torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
        n = rows * cols
        it = [0]

        def rot():
            it[0] += 1
            return xs[it[0] % 3]

        ms, k = time_graphed(lambda: capi.fp8_quantize(rot(), None), 12, min_ms)
        alg = 3.0 * n + 4.0 * rows
        out[f"fp8_per_token_quantize_{rows}x{cols}"] = {"ms": ms, "launches": k, "roofline": hbm_roofline(alg / ms / 1e6, peaks, alg, "fp8_rows_kernel<bf16>")}
        ms, k = time_graphed(lambda: capi.amax(rot()), 12, min_ms)
        out[f"amax_{rows}x{cols}"] = {"ms": ms, "launches": k, "roofline": hbm_roofline(2.0 * n / ms / 1e6, peaks, 2.0 * n, "amax_kernel<bf16>")}
        am = capi.amax(xs[0])
        ms, k = time_graphed(lambda: capi.nvfp4_quantize(rot(), am), 12, min_ms)
        alg = bc.ALG_BYTES_PER_ELEM * n
        out[f"nvfp4_quantize_{rows}x{cols}"] = {"ms": ms, "launches": k,
                                               "roofline": hbm_roofline(alg / ms / 1e6, peaks, alg, "nvfp4_quantize_kernel<bf16, codes>")}
        del xs
    return out


def glue_suite(capi, peaks, min_ms=300.0, tokens=32768, hidden=8192, ffn=28672):
    """The element-wise kernels between the GEMMs of one decoder layer at the stack workload's shape,
    each against the HBM roofline (algorithmic bytes = every operand read once, every result written once)."""
    out = {}
    gu = [torch.randn(tokens, 2 * ffn, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    it = [0]

    def rot(xs):
        it[0] += 1
        return xs[it[0] % len(xs)]

    ms, k = time_device(lambda: capi.silu_mul_fp8_quantize(rot(gu)), min_ms)
    alg = tokens * ffn * (4.0 + 1.0) + 4.0 * tokens
    out[f"silu_mul_fp8_quantize_{tokens}x{ffn}"] = {"ms": ms, "launches": k, "roofline": hbm_roofline(alg / ms / 1e6, peaks, alg, "silu_mul_quant_kernel")}
    del gu
    hs = [torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    ds = [torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    ms, k = time_device(lambda: capi.add_rms_norm_fp8_quantize(rot(hs), rot(ds), w), min_ms)
    alg = tokens * hidden * (2.0 + 2.0 + 2.0 + 1.0) + 4.0 * tokens      # h, delta in; h, codes out
    out[f"add_rms_norm_fp8_quantize_{tokens}x{hidden}"] = {"ms": ms, "launches": k,
                                                           "roofline": hbm_roofline(alg / ms / 1e6, peaks, alg, "add_norm_quant_kernel")}
    return out


# ----------------------------------------------------------------------------- GEMMs
def gemm_case(capi, kind, M, N, K, seed, min_ms=500.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    # several operand sets so that consecutive launches do not find their operands in L2 when they
    # are small enough to fit there
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

    # Every case is timed as a CUDA graph of back-to-back launches over the operand sets, the way a
    # serving loop runs them: below ~100 us a launch issued from Python costs more host time than the
    # kernel takes on the device.  Decode-sized calls (M <= 128) declare their weights static per
    # call (quantized and complete long before), which lets consecutive launches overlap their prologues.
    torch.cuda.synchronize()
    reps = max(nsets, 16 if M <= 2048 else 4)
    with capi.gemm_config(static_weights=(M <= 128)):
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
    ms, n = time_device(graph.replay, min_ms, min_iters=max(4, 50 // reps + 1))
    ms, n = ms / reps, n * reps
    if capi.device_status() != 0:
        raise RuntimeError("device-side wait timed out")
    return ms, n


def gemm_kernel_name(kind, M, N):
    if M <= 128:
        return f"gemm_smallm_kernel<{kind}>"
    if ((M + 255) // 256) * ((N + 255) // 256) >= 74:
        return "gemm_pair_kernel<fp8>" if kind == "fp8" else "gemm_nvf4_pair_kernel"
    return f"gemm_kernel<{kind}>"


def gemm_sweep(capi, peaks, kind, shapes, min_ms=500.0):
    bytes_per_elem = 1.0 if kind == "fp8" else 0.5 + 1.0 / 16
    results = {}
    for idx, (M, N, K) in enumerate(shapes):
        try:
            ms, n = gemm_case(capi, kind, M, N, K, seed=2 + idx, min_ms=min_ms)
        except Exception as exc:  # keep the line even if one shape fails
            results[f"{M}x{N}x{K}"] = {"error": str(exc)[:200]}
            continue
        flops = 2.0 * M * N * K
        byts = (M + N) * K * bytes_per_elem + 2.0 * M * N + (4 * (M + N) if kind == "fp8" else 0) + 2 * N
        tf, gbs = flops / ms / 1e9, byts / ms / 1e6
        entry = {"ms": round(ms, 5), "launches": n, "tflops": round(tf, 1), "GBps": round(gbs, 1)}
        name = gemm_kernel_name(kind, M, N)
        entry["roofline"] = tensor_roofline(tf, peaks, kind, name, flops) if M >= 2048 else hbm_roofline(gbs, peaks, byts, name)
        results[f"{M}x{N}x{K}"] = entry
    return results


def library_comparators(peaks, min_ms=300.0):
    """What the vendor library reaches for the same contraction on this box (cuBLASLt through
    torch._scaled_mm), 8192^3: the fraction of the tensor peak that this box's power cap allows.
    A comparator, not part of the product path; single-GPU runs only (operands in local memory)."""
    out = {}
    M = N = K = 8192
    try:
        a = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(N, K, device="cuda").to(torch.float8_e4m3fn)
        sa, sb = torch.ones(M, 1, device="cuda"), torch.ones(1, N, device="cuda")
        fn = lambda: torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)  # noqa: E731
        ms, n = time_device(fn, min_ms, min_iters=20)
        out["fp8_scaled_mm_8192^3"] = {"ms": ms, "launches": n, "tflops": 2.0 * M * N * K / ms / 1e9}
    except Exception as exc:
        out["fp8_scaled_mm_8192^3"] = {"error": str(exc)[:160]}
    try:
        a = torch.randint(0, 256, (M, K // 2), device="cuda", dtype=torch.uint8).view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 256, (N, K // 2), device="cuda", dtype=torch.uint8).view(torch.float4_e2m1fn_x2)
        sa = torch.full((M * K // 16,), 1.0, device="cuda").to(torch.float8_e4m3fn)
        sb = torch.full((N * K // 16,), 1.0, device="cuda").to(torch.float8_e4m3fn)
        fn = lambda: torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)  # noqa: E731
        ms, n = time_device(fn, min_ms, min_iters=20)
        out["nvfp4_scaled_mm_8192^3"] = {"ms": ms, "launches": n, "tflops": 2.0 * M * N * K / ms / 1e9}
    except Exception as exc:
        out["nvfp4_scaled_mm_8192^3"] = {"error": str(exc)[:160]}
    return out


def attention_case(capi, peaks, min_ms=300.0):
    """FP8 attention of the 70B-shaped stack's prefill (32 sequences of 1024 tokens, 64 q / 8 kv heads of
    128, causal), operands already quantized: device time of b200q_fp8_sdpa alone.  Flops counted as the
    algorithmic 4 B H S^2 D / 2 of a causal attention (the kernel computes Q K^T twice: see its header)."""
    import tensorrt_b200

    lib = tensorrt_b200.load_library()
    B, Hq, Hkv, S, D = 32, 64, 8, 1024, 128
    qc = torch.randint(0, 120, (B, Hq, S, D), dtype=torch.uint8, device="cuda")
    kc = torch.randint(0, 120, (B, Hkv, S, D), dtype=torch.uint8, device="cuda")
    vt = torch.randint(0, 120, (B, Hkv, D, S), dtype=torch.uint8, device="cuda")
    sc = torch.full((1,), 0.01, device="cuda")
    out = torch.empty(B, Hq, S, D, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def fn():
        rc = lib.b200q_fp8_sdpa(qc.data_ptr(), kc.data_ptr(), vt.data_ptr(), sc.data_ptr(), sc.data_ptr(), sc.data_ptr(), out.data_ptr(), 2,
                                B, Hq, Hkv, S, S, S, D, 1.0 / D ** 0.5, 1, stream)
        if rc != 0:
            raise RuntimeError(f"b200q_fp8_sdpa returned {rc}")

    ms, n = time_device(fn, min_ms, min_iters=10)
    flops = 4.0 * B * Hq * S * S * D / 2
    tf = flops / ms / 1e9
    return {"ms": ms, "launches": n, "tflops": tf, "shape": f"B{B} Hq{Hq} Hkv{Hkv} S{S} D{D} causal",
            "roofline": tensor_roofline(tf, peaks, "fp8", "fp8_sdpa_kernel", flops)}


def gated_mlp_case(capi, peaks, min_ms=300.0, tokens=32768, hidden=8192, ffn=28672):
    """The FP8 gated MLP of the stack's shape through `Fp8GatedMlp`: dynamic per-token activation scales (the
    stack's configuration: quantize, gate/up GEMM with the activation in its epilogue, quantize, down GEMM) and
    static per-tensor ones (three launches: the activation's quantizer rides in the epilogue too), against the
    unfused chain (quantize, gate/up GEMM, silu * up + quantize kernel, down GEMM)."""
    import tensorrt_b200 as b200

    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16, generator=g)
    wg, wu = (torch.randn(ffn, hidden, device="cuda", dtype=torch.bfloat16, generator=g) * 0.02 for _ in range(2))
    wd = torch.randn(hidden, ffn, device="cuda", dtype=torch.bfloat16, generator=g) * 0.02
    dyn = b200.Fp8GatedMlp.from_float(wg, wu, wd)
    act = capi.fp8_gemm_silu_mul(*capi.fp8_quantize(x, None), dyn.gu_codes, dyn.gu_scales)
    static = b200.Fp8GatedMlp(dyn.gu_codes, dyn.gu_scales, dyn.down_codes, dyn.down_scales, x.float().abs().max().reshape(1),
                              act.float().abs().max().reshape(1))
    del wg, wu, wd, act

    def unfused():
        xq = capi.fp8_quantize(x, None)
        aq = capi.silu_mul_fp8_quantize(capi.fp8_gemm(xq[0], xq[1], dyn.gu_codes, dyn.gu_scales))
        return capi.fp8_gemm(aq[0], aq[1], dyn.down_codes, dyn.down_scales)

    flops = 2.0 * tokens * hidden * ffn * 3
    out = {"shape": f"{tokens} tokens, hidden {hidden}, ffn {ffn}"}
    variants = (("unfused_dynamic", unfused), ("fused_dynamic", lambda: dyn(x)), ("fused_static", lambda: static(x)))
    # the variants take turns (three rounds each): under the power cap whatever runs later runs warmer and slower
    acc = {name: [0.0, 0] for name, _ in variants}
    for _ in range(3):
        for name, fn in variants:
            ms, k = time_device(fn, min_ms / 3, min_iters=4)
            acc[name][0] += ms * k
            acc[name][1] += k
    for name, (total, k) in acc.items():
        ms = total / k
        out[name] = {"ms": ms, "launches": k, "tflops": flops / ms / 1e9,
                     "roofline": tensor_roofline(flops / ms / 1e9, peaks, "fp8", "gemm_pair_kernel<fp8> (+ glue)", flops)}
    return out


def full_sweep_shapes():
    return [(m, n, k) for (n, k) in SWEEP_NK for m in SWEEP_M]


def extras(capi, peaks, min_ms=500.0):
    """The other two thirds of the metric beside the stack line: quantize GB/s and the full
    quantized-linear GEMM sweep, every entry with its own roofline object, plus the clock record of
    the region they ran in."""
    with bc.ClockSampler(torch.cuda.current_device()) as clocks:
        out = {"quantize": quantize_suite(capi, peaks, min_ms)}
        out["layer_glue"] = glue_suite(capi, peaks)
        for kind in ("fp8", "nvfp4"):
            out[kind + "_gemm"] = gemm_sweep(capi, peaks, kind, full_sweep_shapes(), min_ms)
        try:
            out["fp8_attention"] = attention_case(capi, peaks)
        except Exception as exc:
            out["fp8_attention"] = {"error": str(exc)[:200]}
        try:
            out["fp8_gated_mlp"] = gated_mlp_case(capi, peaks)
        except Exception as exc:
            out["fp8_gated_mlp"] = {"error": str(exc)[:200]}
        out["library"] = library_comparators(peaks)
    out["clocks"] = clocks.summary()
    return out


# ----------------------------------------------------------------------------- workloads
def run_gemm(args, kind):
    from tensorrt_b200 import capi

    torch.cuda.set_device(0)
    peaks = bc.measured_peaks()
    shapes = [tuple(int(v) for v in args.shape.split(","))] if args.shape else full_sweep_shapes()
    with bc.ClockSampler(0) as clocks:
        results = gemm_sweep(capi, peaks, kind, shapes, min_ms=max(100.0, 25.0 * args.steps))
    M, N, K = shapes[-1]
    head = results[f"{M}x{N}x{K}"]
    line = {
        "metric": f"{kind}_quant_linear_gemm_throughput", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
        "steps": head["launches"], "warmup": 3, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "e4m3xe4m3->f32" if kind == "fp8" else "e2m1xe2m1(ue4m3 block scales)->f32",
        "data": "synthetic",
        "config": {"workload": f"{kind} quantized-linear GEMM sweep, headline shape M,N,K = {M},{N},{K}; x ~ N(0,1), "
                               "W ~ N(0,0.02), bias ~ N(0,0.01); operands pre-quantized and resident in HBM",
                   "l2": "operand sets rotate so that sets smaller than L2 are not re-read from L2",
                   "timing": "every shape is timed as a CUDA graph of back-to-back launches (host issue time excluded); "
                             "M <= 128: weights declared static per call (b200q_cfg::static_weights)"},
        "clocks": clocks.summary(), "gpu_launches": head["launches"], "roofline": head["roofline"], "shapes": results,
    }
    print(json.dumps(line))


def quantize_e2e(capi, which, slabs=8, steps=10):
    """The quantize call on HOST buffers: pinned bf16 input -> device, quantize, codes and scales -> pinned host,
    in row slabs on two streams so that the copy-in of slab i + 1 and the copy-out of slab i - 1 run under the
    kernel of slab i (the PCIe link is full duplex).  Returns ms per whole tensor and the bytes each way."""
    rows, cols = (bc.ROWS, bc.COLS) if which == "nvfp4" else (16384, 4096)
    x_host = bc.make_input(1, rows, cols).pin_memory()
    x_dev = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    amax = capi.amax(x_host.cuda())                       # calibrated beforehand, as in the reference's flow
    step = rows // slabs
    outs_host = None
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    d2h = 0

    def once():
        nonlocal outs_host, d2h
        results = []
        for i in range(slabs):
            sl = slice(i * step, (i + 1) * step)
            with torch.cuda.stream(copy_in):
                x_dev[sl].copy_(x_host[sl], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record()
            torch.cuda.current_stream().wait_event(ready)
            out = capi.nvfp4_quantize(x_dev[sl], amax) if which == "nvfp4" else capi.fp8_quantize(x_dev[sl], None)
            done = torch.cuda.Event()
            done.record()
            results.append((out, done))
        if outs_host is None:
            outs_host = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in out] for out, _ in results]
            d2h = sum(t.numel() * t.element_size() for hs in outs_host for t in hs)
        with torch.cuda.stream(copy_out):
            for (out, done), hs in zip(results, outs_host):
                copy_out.wait_event(done)
                for t, h in zip(out, hs):
                    h.copy_(t, non_blocking=True)
        torch.cuda.current_stream().wait_stream(copy_out)
        torch.cuda.synchronize()

    for _ in range(3):
        once()
    import time as _time

    t0 = _time.perf_counter()
    for _ in range(steps):
        once()
    ms = (_time.perf_counter() - t0) * 1e3 / steps       # every call ends with a synchronize: host clock = device + copies
    return ms, x_host.numel() * 2, d2h


def run_quantize(args, which):
    from tensorrt_b200 import capi

    torch.cuda.set_device(0)
    peaks = bc.measured_peaks()
    with bc.ClockSampler(0) as clocks:
        suite = quantize_suite(capi, peaks, min_ms=max(100.0, 25.0 * args.steps))
        e2e_ms, h2d, d2h = quantize_e2e(capi, which)
    key = "nvfp4_quantize_8192x8192_seed1" if which == "nvfp4" else "fp8_per_token_quantize_16384x4096"
    head = suite[key]
    print(json.dumps({
        "metric": f"{which}_quantize_throughput", "value": head["roofline"]["achieved"], "unit": "GB/s", "n_gpus": 1,
        "steps": head["launches"], "warmup": 3, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": key, "l2": "rotating inputs larger than the 126 MB L2"},
        "clocks": clocks.summary(), "gpu_launches": head["launches"], "roofline": head["roofline"],
        "e2e": {"value": head["roofline"]["algorithmic_bytes_per_launch"] / e2e_ms / 1e6, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "path": "pinned host tensor -> device, quantize, codes + scales -> pinned host, 8 row slabs pipelined on two copy streams"},
        "kernels": suite}))


def run_small_cases(args):
    """`--workload small_cases`: a few launches of the element-wise kernels and of the attention kernel on inputs
    of a few hundred MB (larger than L2), for `ncu` captures that end by themselves.  Nothing is timed."""
    from tensorrt_b200 import capi

    torch.cuda.set_device(0)
    tokens, hidden, ffn = 4096, 8192, 28672
    gu = torch.randn(tokens, 2 * ffn, device="cuda", dtype=torch.bfloat16)
    act = torch.randn(tokens, ffn, device="cuda", dtype=torch.bfloat16)
    h = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    d = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    B, Hq, Hkv, S, D = 2, 64, 8, 1024, 128
    q = torch.randn(B, Hq, S, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, device="cuda", dtype=torch.bfloat16)
    am = torch.tensor([4.0], device="cuda")
    for _ in range(2):
        capi.silu_mul_fp8_quantize(gu)
        capi.add_rms_norm_fp8_quantize(h, d, w)
        capi.fp8_quantize(act, None)
        capi.fp8_sdpa(q, k, v, am, am, am, True)
    torch.cuda.synchronize()
    print(json.dumps({"workload": "small_cases", "device_status": capi.device_status(),
                      "cases": {"silu_mul_fp8_quantize": [tokens, 2 * ffn], "add_rms_norm_fp8_quantize": [tokens, hidden],
                                "fp8_quantize": [tokens, ffn], "fp8_sdpa": [B, Hq, Hkv, S, D]}, "launches_each": 2}))


def run(args):
    if args.workload == "small_cases":
        return run_small_cases(args)
    if args.workload == "fp8_gemm":
        run_gemm(args, "fp8")
    elif args.workload == "nvfp4_gemm":
        run_gemm(args, "nvfp4")
    elif args.workload == "fp8_quantize":
        run_quantize(args, "fp8")
    elif args.workload == "nvfp4_quantize":
        run_quantize(args, "nvfp4")
    else:
        raise SystemExit(f"unknown workload {args.workload!r}")
