"""CPU restatement of the quantized-linear hot path (eager semantics).  Test infrastructure.

Parity unpinned for codes and block scales (see the package docstring): the
reference holds no golden vectors for them.  Every choice the reference leaves open is
fixed here, in one place, and the CUDA kernels reproduce exactly this order of IEEE
fp32 operations:

FP8 (E4M3, `tensorrt::quantize_op` with num_bits=8, exponent_bits=4)
  * scale = amax / 448 in fp32 (py/torch_tensorrt/dynamo/conversion/impl/quantize.py:73-104:
    `max_bound = 448`, `scale = torch.divide(amax, max_bound)`); amax == 0 -> scale 1.
  * code  = e4m3_rne(clamp(x_fp32 / scale, -448, +448)); true fp32 division, clamp
    BEFORE the cast (torch's cast gives NaN above 464 instead of saturating).
  * the op returns Q then DQ: (code_as_fp32 * scale) rounded to the input dtype
    (impl/quantize.py:126-138: add_quantize followed by add_dequantize with
    output_type = input dtype).
  * amax may be a scalar (per-tensor, what the reference converter accepts,
    impl/quantize.py:96-100) or have one value per row, shape [rows, 1]
    (per-token activations / per-channel weights: an extension with the same schema).

NVFP4 (`tensorrt::dynamic_block_quantize_op`, num_bits=4, exponent_bits=2,
        scale_num_bits=8, scale_exponent_bits=4, block_size=16)
  * global = (amax / 6) / 448 in fp32, zero replaced by 1
    (impl/dynamic_block_quantize.py:299-308).
  * per 16-element block on the last axis (impl/dynamic_block_quantize.py:59,149-155):
      s_blk = e4m3_rne(min((amax_blk / 6) / global, 448))         stored 8-bit scale
      d     = fp32(s_blk) * global                                 effective divisor
      code  = e2m1_rne(clamp(x_fp32 / d, -6, +6)), ties to the even code;
      a block whose stored scale is zero gets all-zero codes.
  * dequantize = e2m1 * (e4m3 * global) (impl/dynamic_block_quantize.py:201-221: the
    block scale is dequantized by the global scale, the data by that result).
  * two codes per byte, element 2i in the low nibble (matches torch.float4_e2m1fn_x2;
    the reference turns such a uint8 constant into FP4 with the last dim doubled,
    conversion/converter_utils.py:449-470).
  * block scales are stored in the "128x4" swizzled layout the tensor-core
    block-scaled MMA consumes: rows padded to 128, scale columns to 4; tile (rt, ct)
    at byte (rt * n_col_tiles + ct) * 512; inside a tile row r, column c at
    (r % 32) * 16 + (r // 32) * 4 + c.  Padding bytes are zero.

Linear (`aten.linear` fed by Q/DQ, impl/linear.py:40-67): y = x_hat @ W_hat^T + b with
fp32 accumulation, rounded to bf16.

All-reduce (`tensorrt::fused_nccl_all_reduce`, lowering/passes/fuse_distributed_ops.py:57-63):
elementwise sum over ranks (fp32 accumulation, cast to the input dtype).
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = [
    "E4M3_MAX", "E2M1_MAX", "E2M1_VALUES",
    "e4m3_decode_table", "e4m3_encode_np", "e4m3_encode", "e4m3_decode",
    "e2m1_encode", "e2m1_decode",
    "fp8_scale", "fp8_quantize", "fp8_dequantize", "fp8_fake_quant", "row_amax",
    "nvfp4_global_scale", "nvfp4_quantize", "nvfp4_dequantize", "nvfp4_fake_quant",
    "pack_e2m1", "unpack_e2m1", "swizzle_scales", "unswizzle_scales", "swizzled_scale_bytes",
    "quantize_op", "dynamic_block_quantize_op",
    "linear_ref", "fp8_linear_ref", "nvfp4_linear_ref", "rel_l2",
    "all_reduce_ref", "rms_norm_ref", "decoder_layer_ref", "shard_decoder_layer", "fp8_sdpa_ref", "causal_attention_ref",
]

E4M3_MAX = 448.0
E2M1_MAX = 6.0
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


# --------------------------------------------------------------------------- formats
def e4m3_decode_table() -> np.ndarray:
    """All 256 E4M3 (fn: no inf, 0x7F/0xFF = NaN) values, from the format definition:
    1 sign, 4 exponent (bias 7), 3 mantissa bits; subnormals at exponent field 0."""
    out = np.zeros(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        e = (code >> 3) & 0xF
        m = code & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        out[code] = sign * v
    return out


def e4m3_encode_np(x: np.ndarray) -> np.ndarray:
    """Independent numpy E4M3 encoder: round to nearest even, saturate to +-448.
    Used only to cross-check `e4m3_encode` (which goes through torch's cast)."""
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x)
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    # quantum: 2^-9 in the subnormal range, else 2^(floor(log2 a) - 3)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)
    quantum = 2.0 ** (e - 3)
    n = np.rint(a / quantum)  # np.rint is ties-to-even
    v = n * quantum
    # re-derive fields from the rounded value
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(v > 0, v, 1.0)))
    e2 = np.maximum(e2, -6.0)
    is_sub = v < 2.0 ** -6
    mant = np.where(is_sub, v / 2.0 ** -9, (v / 2.0 ** e2 - 1.0) * 8.0)
    expf = np.where(is_sub, 0, e2 + 7)
    code = (expf.astype(np.int64) << 3) | np.rint(mant).astype(np.int64)
    code = np.where(v == 0, 0, code)
    code = code | (sign.astype(np.int64) << 7)
    return code.astype(np.uint8)


def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> E4M3 code bytes: clamp to +-448, then round to nearest even."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_decode(codes: torch.Tensor) -> torch.Tensor:
    return codes.view(torch.float8_e4m3fn).float()


def e2m1_encode(q: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit E2M1 code (uint8 in 0..15): saturate to +-6, round to nearest on
    the grid {0,.5,1,1.5,2,3,4,6}, ties to the even code; bit 3 is the sign
    (negative zero and negatives that round to zero keep their sign bit)."""
    a = q.float().abs()
    idx = torch.zeros_like(a, dtype=torch.uint8)
    # thresholds between neighbours; a tie goes to the even code
    idx += (a > 0.25).to(torch.uint8)
    idx += (a >= 0.75).to(torch.uint8)
    idx += (a > 1.25).to(torch.uint8)
    idx += (a >= 1.75).to(torch.uint8)
    idx += (a > 2.5).to(torch.uint8)
    idx += (a >= 3.5).to(torch.uint8)
    idx += (a > 5.0).to(torch.uint8)
    sign = torch.signbit(q.float()).to(torch.uint8) << 3
    return idx | sign


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    table = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32)
    return table[codes.long()]


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """[..., C] 4-bit codes -> [..., C/2] bytes; element 2i in the low nibble."""
    lo = codes[..., 0::2]
    hi = codes[..., 1::2]
    return (lo | (hi << 4)).to(torch.uint8)


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    lo = packed & 0xF
    hi = packed >> 4
    return torch.stack((lo, hi), dim=-1).flatten(-2)


# --------------------------------------------------------------------------- FP8
def fp8_scale(amax: torch.Tensor) -> torch.Tensor:
    """scale = amax / 448 (impl/quantize.py:76-79,103); zero amax -> scale 1."""
    s = amax.float() / E4M3_MAX
    return torch.where(s == 0, torch.ones_like(s), s)


def row_amax(x: torch.Tensor) -> torch.Tensor:
    """Per-row abs-max as fp32 [rows, 1] (per-token activations, per-channel weights)."""
    return x.float().abs().amax(dim=-1, keepdim=True)


def fp8_quantize(x: torch.Tensor, amax: torch.Tensor):
    """Returns (codes uint8 with x's shape, scale fp32 broadcastable to x)."""
    scale = fp8_scale(amax)
    if scale.numel() > 1:
        scale = scale.reshape(*x.shape[:-1], 1)
    q = x.float() / scale
    return e4m3_encode(q), scale


def fp8_dequantize(codes: torch.Tensor, scale: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    return (e4m3_decode(codes) * scale.float()).to(dtype)


def fp8_fake_quant(x: torch.Tensor, amax: torch.Tensor) -> torch.Tensor:
    codes, scale = fp8_quantize(x, amax)
    return fp8_dequantize(codes, scale, x.dtype)


# --------------------------------------------------------------------------- NVFP4
def nvfp4_global_scale(amax: torch.Tensor) -> torch.Tensor:
    """impl/dynamic_block_quantize.py:299-308: amax / 6 / 448, zero -> 1."""
    g = (amax.float().reshape(()) / E2M1_MAX) / E4M3_MAX
    return torch.where(g == 0, torch.ones_like(g), g)


def swizzled_scale_bytes(rows: int, cols: int) -> int:
    """Size of the swizzled block-scale buffer for a [rows, cols] tensor (cols % 16 == 0)."""
    rt = (rows + 127) // 128
    ct = (cols // 16 + 3) // 4
    return rt * ct * 512


def swizzle_scales(scales: torch.Tensor) -> torch.Tensor:
    """[R, S] uint8 (row-major) -> flat uint8 buffer in the 128x4 tiled layout."""
    R, S = scales.shape
    rt, ct = (R + 127) // 128, (S + 3) // 4
    pad = torch.zeros(rt * 128, ct * 4, dtype=torch.uint8)
    pad[:R, :S] = scales
    # [rt, 4(j: r//32), 32(r%32), ct, 4(c)] -> [rt, ct, 32, 4(j), 4(c)]
    t = pad.view(rt, 4, 32, ct, 4).permute(0, 3, 2, 1, 4)
    return t.contiguous().view(-1)


def unswizzle_scales(buf: torch.Tensor, rows: int, scale_cols: int) -> torch.Tensor:
    rt, ct = (rows + 127) // 128, (scale_cols + 3) // 4
    t = buf.view(rt, ct, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(rt * 128, ct * 4)
    return t[:rows, :scale_cols].contiguous()


def nvfp4_quantize(x: torch.Tensor, amax: torch.Tensor):
    """x [R, C] (C % 16 == 0).  Returns (packed codes uint8 [R, C/2],
    block scales uint8 E4M3 [R, C/16] row-major, global scale fp32 0-dim)."""
    R, C = x.shape
    assert C % 16 == 0, "NVFP4 needs the last dimension to be a multiple of 16"
    g = nvfp4_global_scale(amax)
    xb = x.float().view(R, C // 16, 16)
    a = xb.abs().amax(dim=-1)
    s = ((a / E2M1_MAX) / g).clamp(max=E4M3_MAX)
    s8 = s.to(torch.float8_e4m3fn)
    d = s8.float() * g
    zero = d == 0
    q = xb / torch.where(zero, torch.ones_like(d), d).unsqueeze(-1)
    codes = e2m1_encode(q.clamp(-E2M1_MAX, E2M1_MAX))
    codes = torch.where(zero.unsqueeze(-1), torch.zeros_like(codes), codes)
    return pack_e2m1(codes.view(R, C)), s8.view(torch.uint8), g


def nvfp4_dequantize(packed: torch.Tensor, scales: torch.Tensor, g: torch.Tensor,
                     dtype=torch.float32) -> torch.Tensor:
    """x_hat = e2m1 * (e4m3 * global)  (impl/dynamic_block_quantize.py:201-221)."""
    R = packed.shape[0]
    v = e2m1_decode(unpack_e2m1(packed)).view(R, -1, 16)
    d = e4m3_decode(scales) * g.float()
    return (v * d.unsqueeze(-1)).view(R, -1).to(dtype)


def nvfp4_fake_quant(x: torch.Tensor, amax: torch.Tensor) -> torch.Tensor:
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])  # >3-D inputs are flattened to 2-D (dynamic_block_quantize.py:43-57)
    p, s, g = nvfp4_quantize(x2, amax)
    return nvfp4_dequantize(p, s, g, x.dtype).view(shape)


# --------------------------------------------------------------------------- op-level restatements
def quantize_op(x, amax, num_bits=8, exponent_bits=4, unsigned=False, narrow_range=False):
    """Eager semantics of tensorrt::quantize_op for the FP8 case the hot path uses
    (argument order: tests/py/dynamo/models/test_models_export.py:789)."""
    if num_bits != 8 or exponent_bits != 4:
        raise ValueError(f"oracle covers FP8 E4M3 only, got {num_bits=}, {exponent_bits=}")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"unsupported input dtype {x.dtype}: float32 | float16 | bfloat16")
    return fp8_fake_quant(x, amax)


def dynamic_block_quantize_op(x, block_size, amax, num_bits=4, exponent_bits=2,
                              scale_num_bits=8, scale_exponent_bits=4):
    """Eager semantics of tensorrt::dynamic_block_quantize_op
    (argument order: conversion/aten_ops_converters.py:948-960)."""
    if (num_bits, exponent_bits, scale_num_bits, scale_exponent_bits) != (4, 2, 8, 4) or block_size != 16:
        raise ValueError("oracle covers NVFP4 only: (4,2) codes, (8,4) scales, block 16")
    if x.shape[-1] % 16:
        raise ValueError("last dimension must be a multiple of 16")
    return nvfp4_fake_quant(x, amax)


# --------------------------------------------------------------------------- linear
def linear_ref(x_hat: torch.Tensor, w_hat: torch.Tensor, bias=None) -> torch.Tensor:
    """fp32 y = x_hat @ w_hat^T + b (impl/linear.py:40-67)."""
    y = x_hat.float() @ w_hat.float().t()
    if bias is not None:
        y = y + bias.float()
    return y


def fp8_linear_ref(x, w, bias=None, x_amax=None, w_amax=None) -> torch.Tensor:
    """Per-token activation x per-channel weight FP8 linear, fp32 result.
    Defaults: dynamic row amax for both operands."""
    x2 = x.reshape(-1, x.shape[-1])
    xa = row_amax(x2) if x_amax is None else x_amax
    wa = row_amax(w) if w_amax is None else w_amax
    xc, xs = fp8_quantize(x2, xa)
    wc, ws = fp8_quantize(w, wa)
    y = linear_ref(fp8_dequantize(xc, xs), fp8_dequantize(wc, ws), bias)
    return y.view(*x.shape[:-1], w.shape[0])


def nvfp4_linear_ref(x, w, bias=None, x_amax=None, w_amax=None) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    xa = x2.float().abs().amax() if x_amax is None else x_amax
    wa = w.float().abs().amax() if w_amax is None else w_amax
    y = linear_ref(nvfp4_dequantize(*nvfp4_quantize(x2, xa)),
                   nvfp4_dequantize(*nvfp4_quantize(w, wa)), bias)
    return y.view(*x.shape[:-1], w.shape[0])


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


# --------------------------------------------------------------------------- tensor parallel
def all_reduce_ref(parts, dtype=None) -> torch.Tensor:
    """Sum over ranks in fp32, cast back (fuse_distributed_ops.py:57-63, reduce_op 'sum')."""
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        acc += p.float()
    return acc.to(dtype or parts[0].dtype)


def rms_norm_ref(x, weight, eps=1e-5):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def _qlinear(x, w, mode):
    if mode == "fp8":
        return fp8_linear_ref(x, w)
    if mode == "nvfp4":
        return nvfp4_linear_ref(x, w)
    raise ValueError(mode)


def shard_decoder_layer(layer: dict, rank: int, world: int, n_q: int, n_kv: int, head_dim: int) -> dict:
    """Column-parallel q/k/v/gate/up (weight rows sliced), row-parallel o/down (weight
    columns sliced), as tools/llm/tensor_parallel_llama_export.py:109-125,151-180 does it.
    `wqkv` rows are [q heads | k heads | v heads]; `wgu` rows are [gate | up]."""
    q, kv = n_q * head_dim, n_kv * head_dim
    qs, kvs = q // world, kv // world
    wq, wk, wv = layer["wqkv"][:q], layer["wqkv"][q:q + kv], layer["wqkv"][q + kv:]
    f = layer["wgu"].shape[0] // 2
    fs = f // world
    gate, up = layer["wgu"][:f], layer["wgu"][f:]
    return {
        "norm1": layer["norm1"], "norm2": layer["norm2"],
        "wqkv": torch.cat([wq[rank * qs:(rank + 1) * qs], wk[rank * kvs:(rank + 1) * kvs],
                           wv[rank * kvs:(rank + 1) * kvs]]).contiguous(),
        "wo": layer["wo"][:, rank * qs:(rank + 1) * qs].contiguous(),
        "wgu": torch.cat([gate[rank * fs:(rank + 1) * fs], up[rank * fs:(rank + 1) * fs]]).contiguous(),
        "wdown": layer["wdown"][:, rank * fs:(rank + 1) * fs].contiguous(),
    }


def causal_attention_ref(qkv, n_q: int, n_kv: int, head_dim: int, seq_len: int) -> torch.Tensor:
    """Attention core of one rank's heads on its QKV output [tokens, (n_q + 2 n_kv) * head_dim] (q heads,
    then k heads, then v heads; tokens = batch * seq_len, sequence-major): causal FP8 SDPA (`fp8_sdpa_ref`)
    with each of Q, K, V quantized per tensor at its own abs-max -> [tokens, n_q * head_dim]."""
    t = qkv.shape[0]
    if seq_len <= 0 or t % seq_len:
        raise ValueError(f"{t} tokens are not whole sequences of {seq_len}")
    b, qw, kvw = t // seq_len, n_q * head_dim, n_kv * head_dim
    heads = lambda x, n: x.reshape(b, seq_len, n, head_dim).permute(0, 2, 1, 3).contiguous()  # noqa: E731
    q, k, v = heads(qkv[:, :qw], n_q), heads(qkv[:, qw:qw + kvw], n_kv), heads(qkv[:, qw + kvw:], n_kv)
    out = fp8_sdpa_ref(q, k, v, q.float().abs().max(), k.float().abs().max(), v.float().abs().max(), is_causal=True)
    return out.permute(0, 2, 1, 3).reshape(t, qw).contiguous()


def decoder_layer_ref(h, layer: dict, n_q: int, n_kv: int, head_dim: int, mode: str,
                      world: int = 1, attention: str = "identity", seq_len: int = 0) -> torch.Tensor:
    """One decoder layer of the linear stack, evaluated as `world` tensor-parallel ranks
    whose row-parallel partial outputs are summed (world=1: the plain layer).

    h -> RMSNorm -> QKV linear -> attention core -> O linear (+ all-reduce) -> residual ->
    RMSNorm -> gate/up linear -> silu(gate)*up -> down linear (+ all-reduce) -> residual.
    Attention core: "identity" = the V slice, each kv head repeated n_q/n_kv times to the q width
    (the linear-stack stand-in); "fp8_sdpa" = causal FP8 attention over sequences of `seq_len`
    tokens (h is then [tokens, hidden], sequence-major), every rank on its own heads.
    Each rank quantizes its own activation slice (per-token amax over the local slice for
    FP8; a per-rank tensor amax for NVFP4)."""
    rep = n_q // n_kv
    dt = h.dtype
    x = rms_norm_ref(h, layer["norm1"])
    parts = []
    for r in range(world):
        sh = shard_decoder_layer(layer, r, world, n_q, n_kv, head_dim)
        qkv = _qlinear(x, sh["wqkv"], mode).to(dt)
        kvw = (n_kv // world) * head_dim
        if attention == "fp8_sdpa":
            attn = causal_attention_ref(qkv, n_q // world, n_kv // world, head_dim, seq_len)
        else:
            v = qkv[..., -kvw:]
            attn = v.reshape(*v.shape[:-1], n_kv // world, 1, head_dim).expand(
                *v.shape[:-1], n_kv // world, rep, head_dim).reshape(*v.shape[:-1], -1)
        parts.append(_qlinear(attn.contiguous(), sh["wo"], mode).to(dt))
    h = h + all_reduce_ref(parts, dt)
    x = rms_norm_ref(h, layer["norm2"])
    parts = []
    for r in range(world):
        sh = shard_decoder_layer(layer, r, world, n_q, n_kv, head_dim)
        gu = _qlinear(x, sh["wgu"], mode).to(dt)
        f = gu.shape[-1] // 2
        act = (torch.nn.functional.silu(gu[..., :f].float()) * gu[..., f:].float()).to(dt)
        parts.append(_qlinear(act, sh["wdown"], mode).to(dt))
    return h + all_reduce_ref(parts, dt)


# --------------------------------------------------------------------------- FP8 attention
def fp8_sdpa_ref(q, k, v, amax_q, amax_k, amax_v, is_causal: bool = False, scale=None) -> torch.Tensor:
    """SDPA whose Q, K, V come from `quantize_op(.., 8, 4, ..)` with per-tensor amax, as the reference
    marks and builds it (py/torch_tensorrt/dynamo/lowering/passes/annotate_fp8_sdpa.py:34-76: softmax
    output quantized to FP8 with the fixed scale 1/448; conversion/impl/attention.py:272-337: static
    1/sqrt(D) factor, softmax normalization, lower-right causal mask):
        S = Q_hat K_hat^T * scale;  P = softmax(S);  P_hat = e4m3(P * 448) / 448;  O = P_hat V_hat
    q [B, Hq, Sq, D], k / v [B, Hkv, Sk, D]; query head h reads kv head h // (Hq // Hkv).  fp32 arithmetic
    on the exactly dequantized operands (code x scale in fp32, as a kernel that consumes the FP8 codes
    sees them; the unfused eager graph would round the fake-quantized tensors to the input dtype first,
    which the reference leaves open), result in q's dtype.  Rows with every key masked give zeros."""
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    qh, kh, vh = (fp8_dequantize(*fp8_quantize(t, a)) for t, a in ((q, amax_q), (k, amax_k), (v, amax_v)))
    rep = Hq // Hkv
    kh, vh = kh.repeat_interleave(rep, dim=1), vh.repeat_interleave(rep, dim=1)
    scale = (1.0 / D ** 0.5) if scale is None else scale
    s = (qh @ kh.transpose(-1, -2)) * scale
    if is_causal:
        i = torch.arange(Sq).view(-1, 1)
        j = torch.arange(Sk).view(1, -1)
        s = s.masked_fill(j > i + (Sk - Sq), float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.where(torch.isnan(p), torch.zeros_like(p), p)             # fully masked rows
    p_hat = e4m3_decode(e4m3_encode(p * E4M3_MAX)) / E4M3_MAX
    return (p_hat @ vh).to(q.dtype)
