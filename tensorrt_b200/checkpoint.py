"""Loading ModelOpt-quantized Hugging Face checkpoints straight into the GEMM operand layouts.

On-disk format (what the reference reads in tools/llm/quantize_utils.py:123-151, 181-266):
`hf_quant_config.json` with `{"quantization": {"quant_algo": "FP8" | "NVFP4", ...}}` next to
`*.safetensors` files that hold, per linear `<name>`,

    FP8     <name>.weight          float8_e4m3fn [N, K]
            <name>.weight_scale    fp32 scalar   (weight = codes * weight_scale)
            <name>.input_scale     fp32 scalar   (static activation scale; amax = scale * 448)
    NVFP4   <name>.weight          uint8 [N, K/2], two E2M1 codes per byte (element 2i in the low nibble)
            <name>.weight_scale    float8_e4m3fn [N, K/16] block scales, row-major
            <name>.weight_scale_2  fp32 scalar   (weight = e2m1 * (block scale * weight_scale_2))
            <name>.input_scale     fp32 scalar   (activation global scale; amax = scale * 448 * 6)

The reference dequantizes these weights back to bf16 and lets Q/DQ nodes re-quantize them at
engine-build time (quantize_utils.py:221-266).  Here the stored codes ARE the GEMM operands:
FP8 codes are used as they are, NVFP4 codes too, and only the block scales are rearranged into
the 128 x 4 swizzled tiles the tensor core reads.  Nothing is dequantized or re-quantized.

Tensor-parallel loading takes the reference's plan (tools/llm/tensor_parallel_llama_llm.py:134-157):
"colwise" linears keep rows [rank * N/W, (rank+1) * N/W) of codes and scales, "rowwise" linears
keep the matching slice of K (codes columns / 2, scale columns / 16); `save_rank_shard` writes
what a rank loaded so that the next start reads only its own file, as
examples/distributed_inference/tensor_parallel_simple_example.py:159-177 does for engines.
"""
from __future__ import annotations

import fnmatch
import json
import os

import torch
from torch import nn

from .linear import Fp8Linear, Nvfp4Linear

E4M3_MAX = 448.0
E2M1_MAX = 6.0

# The reference's Llama TP plan: module-name patterns -> sharding style.
LLAMA_TP_PLAN = {
    "*.q_proj": "colwise", "*.k_proj": "colwise", "*.v_proj": "colwise", "*.gate_proj": "colwise", "*.up_proj": "colwise",
    "*.o_proj": "rowwise", "*.down_proj": "rowwise",
}


def load_quantization_config(model_path: str):
    """The "quantization" object of `<model_path>/hf_quant_config.json`, with "model_path" added;
    None when the directory has no such file (same contract as the reference's
    load_quantization_config for a local directory)."""
    path = os.path.join(model_path, "hf_quant_config.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        cfg = json.load(f)["quantization"]
    cfg["model_path"] = model_path
    return cfg


def swizzle_block_scales(scales: torch.Tensor) -> torch.Tensor:
    """Row-major block scales [R, C] (one byte each) -> the tensor core's layout: rows padded to
    128 and columns to 4 with zeros, tiles of 128 x 4 stored row-tile-major, and inside a tile the
    byte of (r, c) at (r % 32) * 16 + (r // 32) * 4 + c.  Returns a flat uint8 tensor."""
    s = scales.view(torch.uint8) if scales.dtype != torch.uint8 else scales
    r, c = s.shape
    rt, ct = (r + 127) // 128, (c + 3) // 4
    padded = torch.zeros(rt * 128, ct * 4, dtype=torch.uint8, device=s.device)
    padded[:r, :c] = s
    # [rt, r // 32, r % 32, ct, c] -> [rt, ct, r % 32, r // 32, c]
    return padded.view(rt, 4, 32, ct, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def _style_for(name: str, plan) -> str | None:
    if not plan:
        return None
    for pattern, style in plan.items():
        if fnmatch.fnmatch(name, pattern):
            if style not in ("colwise", "rowwise"):
                raise ValueError(f"TP style for {pattern!r} must be 'colwise' or 'rowwise', got {style!r}")
            return style
    return None


def _slice(t: torch.Tensor, dim: int, rank: int, world: int, what: str, multiple: int = 1) -> torch.Tensor:
    size = t.shape[dim]
    if size % world or (size // world) % multiple:
        raise ValueError(f"cannot split {what} of extent {size} over {world} ranks in multiples of {multiple}")
    chunk = size // world
    return t.narrow(dim, rank * chunk, chunk).contiguous()


def _read_tensors(model_path: str) -> dict:
    from safetensors import safe_open

    tensors = {}
    for file in sorted(os.listdir(model_path)):
        if file.endswith(".safetensors"):
            with safe_open(os.path.join(model_path, file), framework="pt", device="cpu") as f:
                for name in f.keys():
                    tensors[name] = f.get_tensor(name)
    return tensors


def load_quantized_linears(model_path: str, device="cuda", rank: int = 0, world: int = 1, plan=None,
                           quant_config: dict | None = None, tensors: dict | None = None) -> dict:
    """Every quantized linear of the checkpoint as an `Fp8Linear` / `Nvfp4Linear` on `device`,
    keyed by module name.  `plan` (e.g. LLAMA_TP_PLAN) shards for tensor parallelism; linears the
    plan does not name are replicated.  A row-parallel linear's bias is kept on rank 0 only, so
    that the sum over ranks adds it once."""
    cfg = quant_config or load_quantization_config(model_path)
    if cfg is None:
        raise RuntimeError(f"{model_path}: no hf_quant_config.json")
    algo = cfg.get("quant_algo")
    if algo not in ("FP8", "NVFP4"):
        raise RuntimeError("Only FP8 or NVFP4 quantization is supported")
    tensors = tensors if tensors is not None else _read_tensors(model_path)
    out = {}
    for key in sorted(tensors):
        if not key.endswith(".weight_scale"):
            continue
        name = key[: -len(".weight_scale")]
        if name + ".weight" not in tensors or name + ".input_scale" not in tensors:
            continue  # the reference skips linears with a missing scale (quantize_utils.py:214-219)
        style = _style_for(name, plan) if world > 1 else None
        weight, w_scale = tensors[name + ".weight"], tensors[key]
        in_scale = tensors[name + ".input_scale"].float().reshape(())
        bias = tensors.get(name + ".bias")
        if bias is not None:
            if style == "colwise":
                bias = _slice(bias, 0, rank, world, f"{name}.bias")
            elif style == "rowwise" and rank != 0:
                bias = None
        bias = None if bias is None else bias.to(torch.bfloat16).to(device)
        if algo == "FP8":
            codes = weight.view(torch.uint8)
            if style == "colwise":
                codes = _slice(codes, 0, rank, world, f"{name}.weight rows")
            elif style == "rowwise":
                codes = _slice(codes, 1, rank, world, f"{name}.weight columns", 16)
            scales = w_scale.float().reshape(-1)
            if scales.numel() not in (1, weight.shape[0]):
                raise ValueError(f"{key}: expected a scalar or one scale per output channel, got {tuple(w_scale.shape)}")
            if scales.numel() > 1 and style == "colwise":
                scales = _slice(scales, 0, rank, world, f"{key}")
            out[name] = Fp8Linear(codes.contiguous().to(device), scales.contiguous().to(device), bias,
                                  (in_scale * E4M3_MAX).to(device))
        else:
            scale2_key = name + ".weight_scale_2"
            if scale2_key not in tensors:
                continue
            codes, blk = weight.view(torch.uint8), w_scale.view(torch.uint8)
            if codes.shape[1] * 2 != blk.shape[1] * 16:
                raise ValueError(f"{name}: packed weight {tuple(codes.shape)} and block scales {tuple(blk.shape)} disagree on K")
            if style == "colwise":
                codes = _slice(codes, 0, rank, world, f"{name}.weight rows")
                blk = _slice(blk, 0, rank, world, f"{key} rows")
            elif style == "rowwise":
                blk = _slice(blk, 1, rank, world, f"{key} columns", 2)       # K / world a multiple of 32
                codes = _slice(codes, 1, rank, world, f"{name}.weight columns")
            out[name] = Nvfp4Linear(codes.contiguous().to(device), swizzle_block_scales(blk).to(device),
                                    tensors[scale2_key].float().reshape(1).to(device), bias,
                                    (in_scale * (E4M3_MAX * E2M1_MAX)).to(device))
    return out


def convert_linear_to_b200_quantized(model: nn.Module, hf_quant_config: dict, device="cuda", rank: int = 0, world: int = 1,
                                     plan=None) -> nn.Module:
    """Counterpart of the reference's convert_linear_to_tensorrt_quantized(model, precision,
    hf_quant_config): every nn.Linear of `model` that the checkpoint holds quantized is replaced
    in place by the real-quant layer built from the stored codes."""
    linears = load_quantized_linears(hf_quant_config["model_path"], device, rank, world, plan, hf_quant_config)
    for name, module in list(model.named_modules()):
        if isinstance(module, nn.Linear) and name in linears:
            parent = model
            *path, leaf = name.split(".")
            for part in path:
                parent = getattr(parent, part)
            setattr(parent, leaf, linears[name])
    return model


def save_rank_shard(linears: dict, path: str) -> None:
    """Write the (already sharded, already swizzled) operands of `linears` to one safetensors
    file; `load_rank_shard` restores them without touching the full checkpoint."""
    from safetensors.torch import save_file

    flat, meta = {}, {}
    for name, lin in linears.items():
        meta[name] = "FP8" if isinstance(lin, Fp8Linear) else "NVFP4"
        for buf, t in lin.named_buffers():
            if t is not None:
                flat[f"{name}.{buf}"] = t.detach().cpu().contiguous()
    save_file(flat, path, metadata={"b200q_linears": json.dumps(meta)})


def load_rank_shard(path: str, device="cuda") -> dict:
    from safetensors import safe_open

    out = {}
    with safe_open(path, framework="pt", device="cpu") as f:
        meta = json.loads(f.metadata()["b200q_linears"])
        keys = set(f.keys())
        for name, algo in meta.items():
            def get(buf):
                k = f"{name}.{buf}"
                return f.get_tensor(k).to(device) if k in keys else None
            if algo == "FP8":
                out[name] = Fp8Linear(get("w_codes"), get("w_scales"), get("bias"), get("input_amax"))
            else:
                out[name] = Nvfp4Linear(get("w_codes"), get("w_scales"), get("w_global"), get("bias"), get("input_amax"))
    return out
