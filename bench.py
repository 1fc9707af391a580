#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Default workload (`tp_stack`): the FP8 tensor-parallel decoder linear stack of Llama-3-70B shape
(hidden 8192, 64 q / 8 kv heads of 128, FFN 28672, 80 layers; per-token FP8 activations, per-channel
FP8 weights; QKV and gate/up column-parallel, O and down row-parallel, each followed by the
all-reduce of `tensorrt::fused_nccl_all_reduce`) at TP = --gpus, prefill of 32 x 1024 tokens, seed 4.
A step is one forward of the whole stack over that batch; the token count is fixed as the TP size
grows (strong scaling).  `value` = tokens/s with activations and weights resident in HBM; `e2e` =
the same through `DecoderStack.forward` from pinned host activations with the full bf16 result
copied back to pinned host memory inside the timed region; decode (batch 64, one token) is
reported beside it.  On one GPU the line also carries `extras`: quantize GB/s and the full
quantized-linear GEMM sweep, each entry with its own roofline object (the other two thirds of the
metric), and the CPU baseline.

One JSON line is printed by rank 0.  `--impl reference` times the CPU restatement of the
reference's eager semantics (oracle/) on the host cores for the same metric and workload.
Other workloads: `nvfp4_stack`, `nvfp4_quantize`, `fp8_quantize`, `fp8_gemm`, `nvfp4_gemm`; `small_cases` launches the
element-wise and attention kernels twice on small inputs (for profiler captures, nothing timed).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="tp_stack",
                    choices=["tp_stack", "nvfp4_stack", "nvfp4_quantize", "fp8_quantize", "fp8_gemm", "nvfp4_gemm", "small_cases"])
    ap.add_argument("--no-extras", action="store_true", help="tp_stack on one GPU: skip the quantize / GEMM sweep and the CPU baseline")
    ap.add_argument("--shape", default="", help="M,N,K for the GEMM workloads (default: the whole sweep)")
    ap.add_argument("--micro-batches", type=int, default=0, dest="micro_batches",
                    help="tp_stack: micro-batches of tokens walking the layers on separate streams (exchange / GEMM overlap); "
                         "0 = 4, or 8 at TP >= 8")
    ap.add_argument("--fused", type=int, default=1, help="tp_stack: 1 = fused GEMM + peer-memory all-reduce, 0 = NCCL")
    ap.add_argument("--decode-graph", type=int, default=-1, dest="decode_graph",
                    help="tp_stack: 1 = replay the decode step as a CUDA graph (one GPU only), 0 = issue it launch by launch, "
                         "-1 = graph on one GPU, launch by launch otherwise")
    ap.add_argument("--phase", choices=["all", "prefill", "decode"], default="all",
                    help="tp_stack: time only the prefill or only the decode step (profiling runs)")
    ap.add_argument("--layers", type=int, default=0, help="tp_stack / nvfp4_stack: override the layer count (profiling runs; 0 = the config's)")
    ap.add_argument("--sharded", type=int, default=1,
                    help="tp_stack prefill: 1 = token-sharded residual stream (reduce-scatter + all-gather of FP8 codes), "
                         "0 = all-reduce")
    ap.add_argument("--attention", choices=["identity", "fp8_sdpa"], default="identity",
                    help="tp_stack: attention core between the QKV and O linears: the V-slice stand-in of the linear stack "
                         "(default, the configuration the metric is quoted on) or causal FP8 attention over the 1024-token sequences")
    ap.add_argument("--gate-up-fused", type=int, default=1, dest="gate_up_fused",
                    help="tp_stack: 1 = silu(gate) * up in the epilogue of the gate/up GEMM, 0 = in its own kernel (A/B runs)")
    ap.add_argument("--call-times", type=int, default=0, dest="call_times",
                    help="tp_stack on one GPU: 1 = one extra forward with CUDA events around every library call; "
                         "per-call totals are added to the line as `call_times`")
    ap.add_argument("--slabs", type=int, default=1, help="row slabs per row-parallel linear (all-reduce overlap) in tp_stack")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.workload not in ("tp_stack", "nvfp4_stack"):
            raise SystemExit("--impl reference covers the stack workloads")
        import bench_stack

        bench_stack.run_reference(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.workload in ("tp_stack", "nvfp4_stack"):
        import bench_stack

        bench_stack.run(args)
    else:
        import bench_kernels

        bench_kernels.run(args)


if __name__ == "__main__":
    main()
