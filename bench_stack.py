"""Decoder linear stacks end to end: `bench.py` (default, `--workload tp_stack`) and `--workload nvfp4_stack`.

tp_stack     FP8 (per-token activations, per-channel weights), Llama-3-70B shape (hidden 8192,
             64 q / 8 kv heads of 128, FFN 28672, 80 layers), tensor parallel over --gpus ranks
             (column-parallel QKV / gate-up, row-parallel O / down followed by the all-reduce of
             `tensorrt::fused_nccl_all_reduce`, here fused into the GEMM epilogue over peer memory),
             prefill of 32 x 1024 tokens plus single-token decode steps of batch 64, seed 4.
nvfp4_stack  NVFP4 W4A4, Llama-3-8B shape (hidden 4096, 32 q / 8 kv heads of 128, FFN 14336,
             32 layers), prefill of 8 x 2048 tokens, seed 3; one GPU.

value = prefill tokens/s of the whole job (strong scaling: the token count is fixed as the TP size
grows); decode tokens/s is reported beside it.  Before anything is timed, a 2-layer reduced-width
stack runs through the same code path (same TP size, same fused kernels, same micro-batching) and
is compared with the CPU oracle evaluated as that many ranks; the process exits non-zero when the
comparison fails.  The CPU baseline and `--impl reference` time the oracle's layer arithmetic on
a slab of tokens of ONE full-width layer on the host cores and extrapolate to the whole stack.
"""
from __future__ import annotations

import dataclasses
import json
import os
import time

import torch

import bench_common as bc

PARITY_TOL = 2e-2   # rel-L2 of the bf16 stack output against the oracle (bf16 intermediates round differently)


def workload_string(cfg, batch, seq):
    return (f"{cfg.mode} decoder linear stack hidden {cfg.hidden}, {cfg.n_q}q/{cfg.n_kv}kv x {cfg.head_dim}, ffn {cfg.ffn}, "
            f"{cfg.layers} layers; prefill {batch} x {seq} tokens; random-init weights N(0, 0.02); "
            + ("attention core = identity on the V slice (kv heads repeated to the query width)" if cfg.attention == "identity"
               else "attention core = causal FP8 SDPA per sequence (Q, K, V quantized per tensor)"))


def _config(args):
    from tensorrt_b200.stack import LLAMA3_8B, LLAMA3_70B

    tp = args.workload == "tp_stack"
    cfg = LLAMA3_70B if tp else LLAMA3_8B
    if getattr(args, "layers", 0):
        cfg = dataclasses.replace(cfg, layers=args.layers)   # shortened stack: profiling runs only
    batch, seq = (32, 1024) if tp else (8, 2048)
    if getattr(args, "attention", "identity") != "identity":
        cfg = dataclasses.replace(cfg, attention=args.attention, seq_len=seq)
    return tp, cfg, (batch, seq), (4 if tp else 3)


# ----------------------------------------------------------------------------- parity gate
def parity_check(rank, world, dev, mb, sharded, fused):
    """2 layers, reduced width, same code path and TP size; rank 0 compares with the oracle."""
    from tensorrt_b200 import capi
    from tensorrt_b200.stack import DecoderStack, StackConfig

    cfg = StackConfig(hidden=1024, n_q=16, n_kv=8, head_dim=64, ffn=2048, layers=2, mode="fp8")
    g = torch.Generator().manual_seed(40)
    ws = []
    for _ in range(cfg.layers):
        rnd = lambda r, c: (torch.randn(r, c, generator=g) * 0.02).bfloat16()  # noqa: E731
        ws.append({"norm1": (1 + 0.1 * torch.randn(cfg.hidden, generator=g)).bfloat16(),
                   "norm2": (1 + 0.1 * torch.randn(cfg.hidden, generator=g)).bfloat16(),
                   "wqkv": rnd(cfg.q_width + 2 * cfg.kv_width, cfg.hidden), "wo": rnd(cfg.hidden, cfg.q_width),
                   "wgu": rnd(2 * cfg.ffn, cfg.hidden), "wdown": rnd(cfg.hidden, cfg.ffn)})
    tokens = max(1, mb) * world * 128
    h = torch.randn(tokens, cfg.hidden, generator=g).bfloat16()
    stack = DecoderStack(cfg, [{k: v.to(dev) for k, v in w.items()} for w in ws], rank=rank, world=world,
                         fused_rows=tokens if (world > 1 and fused) else 0)
    y = stack.forward(h.to(dev), mb, sharded)
    y2 = stack.forward(h.to(dev), mb, sharded)           # second pass: reused peer buffers and flag epochs
    torch.cuda.synchronize()
    status = capi.device_status()
    out = {"tol": PARITY_TOL, "tokens": tokens, "layers": cfg.layers, "hidden": cfg.hidden, "world": world, "device_status": status,
           "repeatable": bool(torch.equal(y, y2))}
    if rank == 0:
        import oracle as o

        ref = h
        for w in ws:
            ref = o.decoder_layer_ref(ref, w, cfg.n_q, cfg.n_kv, cfg.head_dim, "fp8", world=world)
        out["rel_l2"] = o.rel_l2(y.float().cpu(), ref.float())
        out["ok"] = bool(out["rel_l2"] <= PARITY_TOL and status == 0 and out["repeatable"])
    del stack
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------- CPU leg (oracle)
_cpu_cache: dict = {}
CPU_ROW_FRACTION = 8      # the CPU sample covers 1/8 of the output rows of each of a layer's four linears


def cpu_layer_sample(cfg, seed, tokens_a=128, tokens_b=1024):
    """The oracle's arithmetic of one full-width layer on the host cores, on a bounded sample: each
    of the layer's four quantized linears (`oracle.fp8_linear_ref` / `nvfp4_linear_ref`: fake-quant
    of activation and weight, fp32 matmul) restricted to 1/8 of its output rows, on two slabs of
    tokens, plus the layer's element-wise glue on the larger slab.  The reference's eager path
    fake-quantizes the weights in every forward, so the cost is  t_weights + tokens * t_token ; the
    two slab sizes separate the terms.  Returns (t_weights, t_token, cores, slabs) for the FULL layer
    (the 1/8 sample multiplied out)."""
    import oracle as o

    torch.set_num_threads(os.cpu_count() or 1)
    key = (cfg.hidden, cfg.ffn, cfg.n_q, cfg.n_kv, cfg.mode, seed)
    if key not in _cpu_cache:
        g = torch.Generator().manual_seed(seed)
        f = CPU_ROW_FRACTION
        rnd = lambda r, c: (torch.randn(r // f, c, generator=g) * 0.02).bfloat16()  # noqa: E731
        _cpu_cache[key] = ([rnd(cfg.q_width + 2 * cfg.kv_width, cfg.hidden), rnd(cfg.hidden, cfg.q_width),
                            rnd(2 * cfg.ffn, cfg.hidden), rnd(cfg.hidden, cfg.ffn)],
                           torch.randn(tokens_b, max(cfg.hidden, cfg.ffn), generator=g).bfloat16())
    weights, acts = _cpu_cache[key]
    linear = o.fp8_linear_ref if cfg.mode == "fp8" else o.nvfp4_linear_ref
    linear(acts[:8, :weights[0].shape[1]], weights[0][:64])      # warm the thread pool
    times = {}
    for n in (tokens_a, tokens_b):
        t0 = time.perf_counter()
        for w in weights:
            linear(acts[:n, :w.shape[1]].contiguous(), w).bfloat16()
        times[n] = time.perf_counter() - t0
    t0 = time.perf_counter()
    ones = torch.ones(cfg.hidden).bfloat16()
    x = acts[:, :cfg.hidden].contiguous()
    o.rms_norm_ref(x, ones)
    o.rms_norm_ref(x + x, ones)
    gu = acts[:, :cfg.ffn].float()
    (torch.nn.functional.silu(gu) * gu).bfloat16()
    glue_per_token = (time.perf_counter() - t0) / tokens_b
    per_token_s = max(0.0, (times[tokens_b] - times[tokens_a]) / (tokens_b - tokens_a))
    t_w_s = max(0.0, times[tokens_a] - tokens_a * per_token_s)
    f = CPU_ROW_FRACTION
    return t_w_s * f, per_token_s * f + glue_per_token, torch.get_num_threads(), (tokens_a, tokens_b)


def cpu_extrapolated(cfg, seed, tokens, repeats=1):
    """tokens/s of the whole stack on the host cores, from the median of `repeats` bounded samples."""
    runs = sorted((cpu_layer_sample(cfg, seed) for _ in range(repeats)), key=lambda r: r[0] + tokens * r[1])
    t_w, per_token, cores, slabs = runs[len(runs) // 2]
    secs = cfg.layers * (t_w + tokens * per_token)
    sample = (f"the four quantized linears of one full-width layer at 1/{CPU_ROW_FRACTION} of their output rows, on slabs of "
              f"{slabs[0]} and {slabs[1]} tokens, plus the layer's element-wise glue: weight fake-quant {t_w:.2f} s per layer and "
              f"forward, {per_token * 1e3:.3f} ms per token and layer (sample multiplied out); extrapolated to {cfg.layers} "
              f"layers x {tokens} tokens = {secs:.0f} s per forward")
    return tokens / secs, cores, sample, secs


def run_reference(args):
    """`bench.py --impl reference`: the CPU oracle on the host cores, rank 0 only; a step is one
    bounded sample (one layer, two token slabs), the value is the extrapolated whole-stack rate."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    tp, cfg, (batch, seq), seed = _config(args)
    if cfg.attention != "identity":
        raise SystemExit("--impl reference times the default attention core (the linear stack the metric is quoted on)")
    tokens = batch * seq
    for _ in range(min(args.warmup, 1)):
        cpu_extrapolated(cfg, seed, tokens)
    vals, t0 = [], time.perf_counter()
    for _ in range(max(1, args.steps)):
        vals.append(cpu_extrapolated(cfg, seed, tokens))
    dt = time.perf_counter() - t0
    vals.sort(key=lambda v: v[0])
    value, cores, sample, secs = vals[len(vals) // 2]
    print(json.dumps({
        "impl": "reference", "metric": "tp_decoder_stack_prefill_throughput" if tp else "nvfp4_decoder_stack_prefill_throughput",
        "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / max(1, args.steps) * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": workload_string(cfg, batch, seq)},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample + " (extrapolated; median of the steps; CPU restatement of the reference's eager "
                                            "semantics: its own implementation lives in packages absent from this image)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ----------------------------------------------------------------------------- GPU arm
def _layer_gemm_ms(capi, cfg, world, tokens):
    """Device time of the four GEMMs of one layer at this rank's shard shapes, all tokens, no exchange."""
    import bench_kernels as bk

    def operands(n, k):
        x = torch.randn(tokens, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.02
        if cfg.mode == "fp8":
            return capi.fp8_quantize(x, None), capi.fp8_quantize(w, capi.row_amax(w))
        return capi.nvfp4_quantize(x, capi.amax(x)), capi.nvfp4_quantize(w, capi.amax(w))

    shapes = [((cfg.q_width + 2 * cfg.kv_width) // world, cfg.hidden), (cfg.hidden, cfg.q_width // world),
              (2 * cfg.ffn // world, cfg.hidden), (cfg.hidden, cfg.ffn // world)]
    total = 0.0
    for n, k in shapes:
        xq, wq = operands(n, k)
        if cfg.mode == "fp8":
            fn = lambda: capi.fp8_gemm(xq[0], xq[1], wq[0], wq[1], None)  # noqa: E731
        else:
            fn = lambda: capi.nvfp4_gemm(xq[0], xq[1], xq[2], wq[0], wq[1], wq[2], None)  # noqa: E731
        ms, _ = bk.time_device(fn, min_ms=100.0, min_iters=5)
        total += ms
        del xq, wq
    return total


def collective_stage_times(capi, stack, cfg, world, rows, iters=20):
    """CUDA-event time of one token-sharded row-parallel linear at this rank's shapes and `rows` tokens
    (one micro-batch), `iters` of them back to back so that the ranks pace each other through the flag
    exchange as in a forward: the GEMM whose epilogue pushes its partial tiles to the owners + the
    owners' reduce, residual add, RMSNorm, FP8 quantize and all-gather of codes, against the same GEMM
    with a local output alone.  Max over ranks, with the algorithmic NVLink bytes each rank sends."""
    rp, layer = stack._fused, stack.layers[0]
    h_shard = torch.zeros(rows // world, cfg.hidden, device="cuda", dtype=torch.bfloat16)
    rp.prepare(rows)

    def loop(fn):
        for _ in range(3):
            fn()
        bc.barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return bc.max_over_ranks(e0.elapsed_time(e1) / iters, world)

    out = {"tokens": rows}
    push_bytes = 2.0 * rows * cfg.hidden * (world - 1) / world
    gather_bytes = (1.0 * rows * cfg.hidden + 4.0 * rows) * (world - 1) / world
    # HBM bytes of the owners' kernel: `world` partials and the residual in, residual and the local copy of the codes out
    reduce_hbm = (rows / world) * cfg.hidden * (2.0 * world + 2.0 + 2.0) + rows * cfg.hidden * 1.0
    for name, k, w in (("o_proj", cfg.q_width // world, layer.wo), ("down_proj", cfg.ffn // world, layer.wdown)):
        x = capi.fp8_quantize(torch.randn(rows, k, device="cuda", dtype=torch.bfloat16), None)

        def fused():
            rp.partials_to_owners(x, w)
            rp.reduce_norm_quantize(h_shard, layer.norm2, cfg.eps)

        both = loop(fused)
        local = loop(lambda: capi.fp8_gemm(x[0], x[1], w[0], w[1], None))
        out[name] = {
            "k_per_rank": k, "gemm_reduce_scatter_plus_reduce_gather_ms": both, "gemm_local_output_ms": local,
            "exchange_and_reduce_ms": both - local,
            "nvlink_bytes_out_per_rank": push_bytes + gather_bytes, "nvlink_ms_at_770GBps": (push_bytes + gather_bytes) / 770e9 * 1e3,
            "reduce_kernel_hbm_bytes": reduce_hbm, "reduce_kernel_hbm_ms_at_measured_peak": reduce_hbm / (bc.measured_peaks()["hbm_gbs"] * 1e9) * 1e3,
        }
        del x
    return out


def call_times(capi, stack, h, mb, sharded):
    """One forward with CUDA events around every call into the library (the C-ABI wrappers of `capi`): ms per
    call kind, summed over the forward, with the call count; GEMMs are keyed by their (M, N, K)."""
    import collections

    import tensorrt_b200.stack as st

    names = ("fp8_gemm", "fp8_gemm_silu_mul", "nvfp4_gemm", "add_rms_norm_fp8_quantize", "silu_mul_fp8_quantize", "silu_mul", "rms_norm",
             "expand_heads", "expand_heads_fp8_quantize", "fp8_quantize", "nvfp4_quantize", "amax", "add")
    records, saved = [], {}

    def wrap(name):
        orig = getattr(capi, name)

        def timed_call(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = orig(*a, **k)
            e1.record()
            key = name
            if name.startswith("fp8_gemm"):
                key = f"{name}({a[0].shape[0]}, {a[2].shape[0]}, {a[0].shape[1]})"
            records.append((key, e0, e1))
            return r

        saved[name] = (orig, st.CudaBackend.__dict__.get(name))
        setattr(capi, name, timed_call)
        if name in st.CudaBackend.__dict__:
            setattr(st.CudaBackend, name, staticmethod(timed_call))

    for n in names:
        wrap(n)
    try:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stack.forward(h, mb, sharded)
        e1.record()
        torch.cuda.synchronize()
    finally:
        for n, (orig, static) in saved.items():
            setattr(capi, n, orig)
            if static is not None:
                setattr(st.CudaBackend, n, static)
    agg = collections.defaultdict(lambda: [0, 0.0])
    for key, a, b in records:
        agg[key][0] += 1
        agg[key][1] += a.elapsed_time(b)
    return {"forward_ms": e0.elapsed_time(e1),
            "calls": {k: {"n": v[0], "ms_total": v[1], "ms_each": v[1] / v[0]} for k, v in sorted(agg.items(), key=lambda kv: -kv[1][1])}}


def run(args):
    from tensorrt_b200 import capi
    from tensorrt_b200.stack import DecoderStack, random_layer_weights

    rank, world, local = bc.dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    tp, cfg, (batch, seq), seed = _config(args)
    phase = getattr(args, "phase", "all") if tp else "all"
    if not tp and world > 1:
        raise SystemExit("nvfp4_stack is a single-GPU workload; use tp_stack for --gpus > 1")
    want_graph = getattr(args, "decode_graph", -1)
    pull = bool(world > 1 and args.fused and cfg.mode == "fp8")     # decode steps: pull all-reduce over peer memory, no NCCL in the step
    if want_graph > 0 and world > 1 and not pull:
        raise SystemExit("--decode-graph 1 is refused at TP > 1 with NCCL all-reduces inside the step: capturing those is not supported")
    tokens = batch * seq
    mb = args.micro_batches if world > 1 else 1
    if mb <= 0:
        mb = 8 if world >= 8 else 4                      # measured best: 4 at TP 2, 8 at TP 8
    sharded = bool(world > 1 and args.sharded and cfg.mode == "fp8")
    fused = bool(world > 1 and args.fused)

    parity = None
    if tp:
        parity = parity_check(rank, world, dev, min(mb, 2) if world > 1 else 1, sharded, fused)
        if rank == 0 and not parity["ok"]:
            print(json.dumps({"metric": "tp_decoder_stack_prefill_throughput", "parity": parity, "error": "parity check failed"}))
            raise SystemExit(3)

    t0 = time.time()
    from tensorrt_b200.stack import CudaBackend

    stack = DecoderStack(cfg, random_layer_weights(cfg, seed, device=dev), rank=rank, world=world,
                         backend=CudaBackend(cfg.mode, fuse_gate_up=bool(getattr(args, "gate_up_fused", 1))),
                         slabs=args.slabs if world > 1 else 1, fused_rows=tokens if fused else 0, pull_rows=64 if pull else 0)
    torch.cuda.synchronize()
    build_s = time.time() - t0

    g = torch.Generator().manual_seed(seed)
    h_host = torch.randn(batch, seq, cfg.hidden, generator=g).bfloat16().pin_memory()
    y_host = torch.empty_like(h_host).pin_memory()
    h = h_host.to(dev)
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    if cfg.mode == "nvfp4":
        stack.calibrate(h)  # static activation amax in front of every linear, as after calibration

    ms = e2e_ms = float("nan")
    e2e_steps = max(1, min(steps, 3))
    with bc.ClockSampler(local) as clocks:
        if phase != "decode":
            ms = bc.timed(lambda i: stack.forward(h, mb, sharded), steps, warmup, world)
    status = capi.device_status()

    x_dev = torch.empty_like(h) if world > 1 else None

    def e2e(i):
        # the request lives in ONE host process: rank 0 copies it in and the other ranks get it over NVLink
        # (a broadcast on the process group); every rank ends up with the complete result, rank 0 copies it out
        if world == 1:
            x = h_host.to(dev, non_blocking=True)
        else:
            import torch.distributed as dist

            if rank == 0:
                x_dev.copy_(h_host, non_blocking=True)
            dist.broadcast(x_dev, src=0)
            x = x_dev
        y = stack.forward(x, mb, sharded)
        if rank == 0:
            y_host.copy_(y, non_blocking=True)           # the whole [tokens, hidden] bf16 result back to pinned host memory
        torch.cuda.current_stream().synchronize()

    if phase != "decode":
        e2e_ms = bc.timed(e2e, e2e_steps, 1, world)

    decode = None
    if tp and phase != "prefill":
        hd = torch.randn(64, 1, cfg.hidden, generator=g).bfloat16().to(dev)
        dsteps = 20
        decode_fn = lambda: stack(hd)  # noqa: E731
        graphed = False
        if want_graph < 0:
            want_graph = 1 if (world == 1 or pull) else 0
        if want_graph:
            # a decode step is ~700 short launches: issuing them from Python costs more than running
            # them, so the step is replayed as one CUDA graph, the way a serving loop runs it (at TP > 1
            # only with the pull all-reduce, whose launches are this library's own kernels)
            for _ in range(2):
                stack(hd)
            torch.cuda.synchronize()
            bc.barrier(world)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    stack(hd)
            torch.cuda.current_stream().wait_stream(side)
            decode_fn, graphed = graph.replay, True
        dms = bc.timed(lambda i: decode_fn(), dsteps, 3, world)
        decode = {"tokens_per_s": 64 * dsteps / (dms * 1e-3), "ms_per_step": dms / dsteps, "batch": 64, "cuda_graph": graphed,
                  "all_reduce": "pull over peer memory, fused with residual add + RMSNorm + FP8 quantize" if pull else ("NCCL" if world > 1 else "none"),
                  "weight_bytes_per_rank": cfg.weights_per_layer() * cfg.layers // world,
                  "weight_stream_GBps_per_rank": cfg.weights_per_layer() * cfg.layers / world / (dms / dsteps * 1e-3) / 1e9,
                  "frac_of_measured_hbm": cfg.weights_per_layer() * cfg.layers / world / (dms / dsteps * 1e-3) / 1e9
                  / bc.measured_peaks()["hbm_gbs"]}
    status = status or capi.device_status()

    peaks = bc.measured_peaks()
    flops = cfg.flops_per_token() * tokens
    scale = 2.0 if cfg.mode == "fp8" else 4.0
    tflops = flops / (ms / steps * 1e-3) / 1e12
    per_layer_ms = ms / steps / cfg.layers
    breakdown = None
    if phase != "decode":
        # the limiter, from numbers of this run: GEMM-only time of a layer at this rank's shapes
        # against the measured time per layer; the algorithmic NVLink bytes of the exchange beside it
        gemm_ms = _layer_gemm_ms(capi, cfg, world, tokens)
        t_n = tokens * cfg.hidden
        nvlink_out = (2 * 2 * t_n * (world - 1) / world + (2 * t_n * (world - 1) / world if sharded else 2 * 2 * t_n * (world - 1) / world)) if world > 1 else 0
        breakdown = {"ms_per_layer": per_layer_ms, "gemm_only_ms_per_layer": gemm_ms,
                     "exchange_and_glue_exposed_ms_per_layer": per_layer_ms - gemm_ms,
                     "nvlink_bytes_out_per_layer_per_rank": nvlink_out,
                     "nvlink_ms_per_layer_at_770GBps": nvlink_out / 770e9 * 1e3,
                     "limiter": "gemm" if gemm_ms >= 0.8 * per_layer_ms else "exchange + glue not hidden under the GEMMs"}
        if sharded and fused:
            breakdown["collective_stages"] = collective_stage_times(capi, stack, cfg, world, tokens // mb)
    # launches of this library per layer and micro-batch: norm + quantize, QKV GEMM, head expansion + quantize, O GEMM,
    # norm + quantize, gate/up GEMM (activation in its epilogue), quantize, down GEMM; the token-sharded form replaces
    # the two norm kernels by a flag exchange + reduce / norm / quantize / gather pair each
    kernels_per_layer = 10 if (world > 1 and sharded and fused) else 8
    launches = steps * (cfg.layers * kernels_per_layer * (mb if world > 1 else 1) + 2)
    line = {
        "metric": "tp_decoder_stack_prefill_throughput" if tp else "nvfp4_decoder_stack_prefill_throughput",
        "value": tokens * steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "e4m3" if cfg.mode == "fp8" else "e2m1 (nvfp4)", "data": "synthetic",
        "config": {"workload": workload_string(cfg, batch, seq)
                               + ("; activation amax calibrated once (static quantizer input)" if cfg.mode == "nvfp4" else ""),
                   "parallelism": f"tp{world}", "micro_batches": mb, "slabs": args.slabs if world > 1 else 1,
                   "residual_stream": "token-sharded (reduce-scatter, norm + quantize on owned tokens, all-gather of FP8 codes)" if sharded else "replicated",
                   "row_parallel": ("fused GEMM reduce-scatter epilogue + peer-memory reduce/all-gather" if fused
                                    else ("NCCL all-reduce" if world > 1 else "none")),
                   "l2": "weights + activations per forward far exceed the 126 MB L2"},
        "clocks": clocks.summary(), "build_seconds": round(build_s, 1), "device_status": status,
        "gpu_launches": launches,
        "e2e": {"value": tokens * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h_host.numel() * 2,
                "d2h_bytes_per_step": y_host.numel() * 2, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "path": "pinned host bf16 activations -> device"
                        + (" of rank 0 -> broadcast to the ranks over NVLink" if world > 1 else "")
                        + ", DecoderStack.forward, bf16 result -> pinned host" + (" of rank 0" if world > 1 else "")},
        "model_tflops": tflops,
        "roofline": {"bound": "tensor", "achieved": tflops / world, "peak": peaks["bf16_tflops_sustained"] * scale, "unit": "TFLOP/s",
                     "frac": tflops / world / (peaks["bf16_tflops_sustained"] * scale),
                     "peak_source": f"{peaks['source']} sustained cuBLAS bf16 x{int(scale)} per GPU; GEMM flops only, per GPU, "
                                    "over the whole step (glue and exchange kernels included in the time)",
                     "traffic": None, "kernel": "gemm_pair_kernel<fp8>" if cfg.mode == "fp8" else "gemm_nvf4_pair_kernel",
                     "algorithmic_flops_per_step_per_gpu": flops / world},
    }
    if getattr(args, "call_times", 0) and world == 1 and phase != "decode":
        line["call_times"] = call_times(capi, stack, h, mb, sharded)
    if parity is not None:
        line["parity"] = parity
    if breakdown is not None:
        line["per_layer"] = breakdown
    if decode:
        line["decode"] = decode
    if rank == 0 and world == 1 and not args.no_extras:
        value, cores, sample, _ = cpu_extrapolated(cfg, seed, tokens, repeats=7)
        line["cpu_baseline"] = {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample + " (extrapolated)"}
        del stack
        torch.cuda.empty_cache()
        import bench_kernels as bk

        line["extras"] = bk.extras(capi, peaks)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
