"""Python calls straight through the C ABI (include/b200q.h) on torch CUDA tensors.

torch is used for device memory and streams only; every function below hands raw device
pointers to `libb200q.so`.  These are the calls the GPU parity tests exercise.
"""
from __future__ import annotations

import contextlib
import contextvars

import torch

from ._lib import cfg_ref, check, load

_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _dt(x: torch.Tensor) -> int:
    try:
        return _DTYPE[x.dtype]
    except KeyError:
        raise ValueError(f"received an input of {x.dtype} type. Supported types: float32 | float16 | bfloat16") from None


def _stream(x: torch.Tensor) -> int:
    return torch.cuda.current_stream(x.device).cuda_stream


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("b200q operates on CUDA tensors only; there is no CPU implementation")


def _rows_cols(x: torch.Tensor):
    cols = x.shape[-1]
    return (x.numel() // cols if cols else 0), cols


def _ptr(t):
    return None if t is None else t.data_ptr()


_amax_ws: dict = {}


def amax_workspace(device) -> torch.Tensor:
    """Zero-initialised workspace for b200q_amax, one per (device, stream)."""
    key = (torch.device(device).index, torch.cuda.current_stream(device).cuda_stream)
    ws = _amax_ws.get(key)
    if ws is None:
        ws = torch.zeros(load().b200q_amax_workspace_bytes(), dtype=torch.uint8, device=device)
        _amax_ws[key] = ws
    return ws


def amax(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x)
    x = x.contiguous()
    out = torch.zeros((), dtype=torch.float32, device=x.device)
    if x.numel() == 0:
        return out
    ws = amax_workspace(x.device)
    with torch.cuda.device(x.device):
        check(load().b200q_amax(x.data_ptr(), _dt(x), x.numel(), out.data_ptr(), ws.data_ptr(), ws.numel(), _stream(x)),
              "b200q_amax")
    return out


def row_amax(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x)
    x = x.contiguous()
    rows, cols = _rows_cols(x)
    out = torch.empty(rows, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(load().b200q_row_amax(x.data_ptr(), _dt(x), rows, cols, out.data_ptr(), _stream(x)), "b200q_row_amax")
    return out.view(*x.shape[:-1], 1)


def _amax_arg(x, amax_t, rows):
    if amax_t is None:
        return None, 0
    a = amax_t.to(device=x.device, dtype=torch.float32).contiguous()
    n = a.numel()
    if n != 1 and n != rows:
        raise ValueError(f"amax must hold one value or one per row ({rows}), got shape {tuple(amax_t.shape)}")
    return a, n


def fp8_quantize(x: torch.Tensor, amax_t: torch.Tensor | None = None):
    """-> (codes uint8 like x, scales fp32 [1] or [rows]).  amax_t None = dynamic per-row."""
    _need_cuda(x, amax_t)
    x = x.contiguous()
    rows, cols = _rows_cols(x)
    a, n = _amax_arg(x, amax_t, rows)
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(1 if n == 1 else rows, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(load().b200q_fp8_quantize(x.data_ptr(), _dt(x), rows, cols, _ptr(a), n, codes.data_ptr(), scales.data_ptr(),
                                        _stream(x)), "b200q_fp8_quantize")
    return codes, scales


def fp8_fake_quantize(x: torch.Tensor, amax_t: torch.Tensor | None = None) -> torch.Tensor:
    _need_cuda(x, amax_t)
    x = x.contiguous()
    rows, cols = _rows_cols(x)
    a, n = _amax_arg(x, amax_t, rows)
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(load().b200q_fp8_fake_quantize(x.data_ptr(), _dt(x), rows, cols, _ptr(a), n, out.data_ptr(), _stream(x)),
              "b200q_fp8_fake_quantize")
    return out


def fp8_dequantize(codes: torch.Tensor, scales: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    _need_cuda(codes, scales)
    codes = codes.contiguous()
    rows, cols = _rows_cols(codes)
    out = torch.empty(codes.shape, dtype=dtype, device=codes.device)
    with torch.cuda.device(codes.device):
        check(load().b200q_fp8_dequantize(codes.data_ptr(), scales.data_ptr(), scales.numel(), rows, cols, out.data_ptr(),
                                          _DTYPE[dtype], _stream(codes)), "b200q_fp8_dequantize")
    return out


def nvfp4_scale_bytes(rows: int, cols: int) -> int:
    return load().b200q_nvfp4_scale_bytes(rows, cols)


def nvfp4_quantize(x: torch.Tensor, amax_t: torch.Tensor):
    """-> (packed codes uint8 [.., cols/2], swizzled E4M3 block scales uint8 [bytes], global scale fp32 0-dim)."""
    _need_cuda(x, amax_t)
    x = x.contiguous()
    rows, cols = _rows_cols(x)
    if cols % 16:
        raise ValueError(f"last dimension ({cols}) must be a multiple of the block size 16")
    a = amax_t.to(device=x.device, dtype=torch.float32).reshape(1)
    codes = torch.empty(*x.shape[:-1], cols // 2, dtype=torch.uint8, device=x.device)
    scales = torch.empty(nvfp4_scale_bytes(rows, cols), dtype=torch.uint8, device=x.device)
    g = torch.empty((), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(load().b200q_nvfp4_quantize(x.data_ptr(), _dt(x), rows, cols, a.data_ptr(), codes.data_ptr(),
                                          scales.data_ptr(), g.data_ptr(), _stream(x)), "b200q_nvfp4_quantize")
    return codes, scales, g


def nvfp4_fake_quantize(x: torch.Tensor, amax_t: torch.Tensor) -> torch.Tensor:
    _need_cuda(x, amax_t)
    x = x.contiguous()
    rows, cols = _rows_cols(x)
    if cols % 16:
        raise ValueError(f"last dimension ({cols}) must be a multiple of the block size 16")
    a = amax_t.to(device=x.device, dtype=torch.float32).reshape(1)
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(load().b200q_nvfp4_fake_quantize(x.data_ptr(), _dt(x), rows, cols, a.data_ptr(), out.data_ptr(), _stream(x)),
              "b200q_nvfp4_fake_quantize")
    return out


def nvfp4_dequantize(codes, scales, g, dtype=torch.float32) -> torch.Tensor:
    _need_cuda(codes, scales, g)
    codes = codes.contiguous()
    rows, half = _rows_cols(codes)
    out = torch.empty(*codes.shape[:-1], half * 2, dtype=dtype, device=codes.device)
    with torch.cuda.device(codes.device):
        check(load().b200q_nvfp4_dequantize(codes.data_ptr(), scales.data_ptr(), g.data_ptr(), rows, half * 2,
                                            out.data_ptr(), _DTYPE[dtype], _stream(codes)), "b200q_nvfp4_dequantize")
    return out


# Per-call GEMM options (struct b200q_cfg).  `gemm_config` sets the defaults the GEMM wrappers below
# use inside a `with` block of the calling thread / task; nothing is process-wide.
_gemm_cfg = contextvars.ContextVar("b200q_gemm_cfg", default=(0, False))


@contextlib.contextmanager
def gemm_config(tile_n: int | None = None, static_weights: bool | None = None):
    """Defaults for `fp8_gemm` / `nvfp4_gemm` calls made inside the block by this thread:
    `tile_n` forces a kernel / tile shape (b200q_cfg::tile_n), `static_weights` promises that the
    weight operands were complete on the device before the call (b200q_cfg::static_weights)."""
    cur = _gemm_cfg.get()
    token = _gemm_cfg.set((cur[0] if tile_n is None else int(tile_n), cur[1] if static_weights is None else bool(static_weights)))
    try:
        yield
    finally:
        _gemm_cfg.reset(token)


def _cfg(tile_n, static_weights):
    cur = _gemm_cfg.get()
    return cfg_ref(cur[0] if tile_n is None else tile_n, cur[1] if static_weights is None else static_weights)


def _gemm_out(out, shape, device):
    if out is None:
        return torch.empty(shape, dtype=torch.bfloat16, device=device)
    if tuple(out.shape) != tuple(shape) or out.dtype != torch.bfloat16 or not out.is_contiguous() or out.device != device:
        raise ValueError(f"out must be a contiguous bf16 tensor of shape {tuple(shape)} on {device}")
    return out


def fp8_gemm(a_codes, a_scales, b_codes, b_scales, bias=None, tile_n=None, static_weights=None, out=None) -> torch.Tensor:
    """bf16 [.., N] = dequant(a [.., K]) @ dequant(b [N, K])^T + bias (into `out` when given)."""
    _need_cuda(a_codes, a_scales, b_codes, b_scales, bias)
    a_codes, b_codes = a_codes.contiguous(), b_codes.contiguous()
    N, K = b_codes.shape
    M = a_codes.numel() // K
    out = _gemm_out(out, (*a_codes.shape[:-1], N), a_codes.device)
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    with torch.cuda.device(a_codes.device):
        check(load().b200q_fp8_gemm(a_codes.data_ptr(), a_scales.data_ptr(), a_scales.numel(), b_codes.data_ptr(),
                                    b_scales.data_ptr(), b_scales.numel(), _ptr(bias), out.data_ptr(), M, N, K,
                                    _stream(a_codes), _cfg(tile_n, static_weights)), "b200q_fp8_gemm")
    return out


def fp8_gemm_silu_mul(a_codes, a_scales, b_codes, b_scales, bias=None, out=None) -> torch.Tensor:
    """Gate/up linear with the activation in the GEMM epilogue: b [2F, K] = F gate rows then F up rows
    (F a multiple of 128) -> bf16 [.., F] = silu(g) * u, the same bits as `silu_mul(fp8_gemm(..))`."""
    _need_cuda(a_codes, a_scales, b_codes, b_scales, bias)
    a_codes, b_codes = a_codes.contiguous(), b_codes.contiguous()
    k = a_codes.shape[-1]
    m = a_codes.numel() // max(k, 1)
    n = b_codes.shape[0]
    if b_codes.dim() != 2 or b_codes.shape[1] != k or n % 256:
        raise ValueError(f"b must be [2F, {k}] with F a multiple of 128, got {tuple(b_codes.shape)}")
    a_scales, b_scales = a_scales.float().contiguous(), b_scales.float().contiguous()
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    out = _gemm_out(out, tuple(a_codes.shape[:-1]) + (n // 2,), a_codes.device)
    with torch.cuda.device(a_codes.device):
        check(load().b200q_fp8_gemm_silu_mul(a_codes.data_ptr(), a_scales.data_ptr(), a_scales.numel(), b_codes.data_ptr(),
                                             b_scales.data_ptr(), b_scales.numel(), _ptr(bias), out.data_ptr(), m, n, k,
                                             _stream(a_codes), None), "b200q_fp8_gemm_silu_mul")
    return out


def fp8_gemm_silu_mul_quantize(a_codes, a_scales, b_codes, b_scales, act_amax, bias=None):
    """`fp8_gemm_silu_mul` with the activation's static per-tensor FP8 quantizer in the epilogue as well:
    -> (E4M3 codes [.., F] uint8, scale [1] = act_amax / 448), the same bits as quantizing its bf16 result
    with `fp8_quantize(.., act_amax)`."""
    _need_cuda(a_codes, a_scales, b_codes, b_scales, bias, act_amax)
    a_codes, b_codes = a_codes.contiguous(), b_codes.contiguous()
    k = a_codes.shape[-1]
    m = a_codes.numel() // max(k, 1)
    n = b_codes.shape[0]
    if b_codes.dim() != 2 or b_codes.shape[1] != k or n % 256:
        raise ValueError(f"b must be [2F, {k}] with F a multiple of 128, got {tuple(b_codes.shape)}")
    if act_amax.numel() != 1:
        raise ValueError("act_amax must hold one value (a static per-tensor amax)")
    a_scales, b_scales = a_scales.float().contiguous(), b_scales.float().contiguous()
    act_amax = act_amax.float().reshape(1).contiguous()
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    codes = torch.empty(tuple(a_codes.shape[:-1]) + (n // 2,), dtype=torch.uint8, device=a_codes.device)
    scale = torch.empty(1, dtype=torch.float32, device=a_codes.device)
    with torch.cuda.device(a_codes.device):
        check(load().b200q_fp8_gemm_silu_mul_quantize(a_codes.data_ptr(), a_scales.data_ptr(), a_scales.numel(), b_codes.data_ptr(),
                                                      b_scales.data_ptr(), b_scales.numel(), _ptr(bias), act_amax.data_ptr(),
                                                      codes.data_ptr(), scale.data_ptr(), m, n, k, _stream(a_codes), None),
              "b200q_fp8_gemm_silu_mul_quantize")
    return codes, scale


def nvfp4_gemm(a_codes, a_scales, a_global, b_codes, b_scales, b_global, bias=None, tile_n=None, static_weights=None,
               out=None) -> torch.Tensor:
    _need_cuda(a_codes, a_scales, a_global, b_codes, b_scales, b_global, bias)
    a_codes, b_codes = a_codes.contiguous(), b_codes.contiguous()
    N, half = b_codes.shape
    K = half * 2
    M = a_codes.numel() // half
    out = _gemm_out(out, (*a_codes.shape[:-1], N), a_codes.device)
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    with torch.cuda.device(a_codes.device):
        check(load().b200q_nvfp4_gemm(a_codes.data_ptr(), a_scales.data_ptr(), a_global.data_ptr(), b_codes.data_ptr(),
                                      b_scales.data_ptr(), b_global.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K,
                                      _stream(a_codes), _cfg(tile_n, static_weights)), "b200q_nvfp4_gemm")
    return out


def fp8_sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, amax_q, amax_k, amax_v, is_causal: bool = False,
             scale: float | None = None) -> torch.Tensor:
    """FP8 attention on q [B, Hq, Sq, D], k / v [B, Hkv, Sk, D] (bf16 / fp16 / fp32) with per-tensor amax
    each: Q, K, V are quantized to E4M3 (V transposed per head on the way), the softmax output is quantized
    with the fixed scale 1/448, both contractions run on FP8 tensor cores; result in q's dtype."""
    import math

    _need_cuda(q, k, v)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4 or k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3]:
        raise ValueError(f"expected q [B, Hq, Sq, D] and k, v [B, Hkv, Sk, D], got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    B, Hq, Sq, D = q.shape
    _, Hkv, Sk, _ = k.shape
    if Hq % Hkv or D % 16 or D > 128:
        raise ValueError(f"need Hq % Hkv == 0 and a head dimension that is a multiple of 16 up to 128, got Hq={Hq}, Hkv={Hkv}, D={D}")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    dev = q.device
    amaxes = [a.to(device=dev, dtype=torch.float32).reshape(1) for a in (amax_q, amax_k, amax_v)]
    qc, qs = fp8_quantize(q, amaxes[0])
    kc, ks = fp8_quantize(k, amaxes[1])
    stride = (Sk + 15) // 16 * 16
    vt = torch.empty(B, Hkv, D, max(stride, 16), dtype=torch.uint8, device=dev)
    vs = torch.empty(1, dtype=torch.float32, device=dev)
    out = torch.empty_like(q)
    lib = load()
    with torch.cuda.device(dev):
        check(lib.b200q_fp8_quantize_transpose(v.data_ptr(), _dt(v), B * Hkv, Sk, D, amaxes[2].data_ptr(), vt.data_ptr(), max(stride, 16),
                                               vs.data_ptr(), _stream(q)), "b200q_fp8_quantize_transpose")
        if Sk == 0:
            vs.fill_(1.0)
        check(lib.b200q_fp8_sdpa(qc.data_ptr(), kc.data_ptr(), vt.data_ptr(), qs.data_ptr(), ks.data_ptr(), vs.data_ptr(), out.data_ptr(),
                                 _dt(q), B, Hq, Hkv, Sq, Sk, max(stride, 16), D, float(scale if scale is not None else 1.0 / math.sqrt(D)),
                                 1 if is_causal else 0, _stream(q)), "b200q_fp8_sdpa")
    return out


def _bf16(*ts):
    for t in ts:
        if t.dtype != torch.bfloat16:
            raise ValueError(f"expected bfloat16, got {t.dtype}")


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    _need_cuda(x, weight)
    _bf16(x, weight)
    x = x.contiguous()
    rows, cols = _rows_cols(x)
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(load().b200q_rms_norm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, cols, eps, _stream(x)), "b200q_rms_norm")
    return out


def add_rms_norm_fp8_quantize(h: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float = 1e-5):
    """-> (h + delta (h itself when delta is None), FP8 codes of rms_norm(h + delta), per-token scales)."""
    _need_cuda(h, delta, weight)
    _bf16(h, weight)
    h = h.contiguous()
    rows, cols = _rows_cols(h)
    h_out = h
    if delta is not None:
        _bf16(delta)
        delta = delta.contiguous()
        h_out = torch.empty_like(h)
    codes = torch.empty(h.shape, dtype=torch.uint8, device=h.device)
    scales = torch.empty(rows, dtype=torch.float32, device=h.device)
    with torch.cuda.device(h.device):
        check(load().b200q_add_rms_norm_fp8_quantize(h.data_ptr(), _ptr(delta), weight.data_ptr(), h_out.data_ptr(), codes.data_ptr(),
                                                     scales.data_ptr(), rows, cols, eps, _stream(h)), "b200q_add_rms_norm_fp8_quantize")
    return h_out, codes, scales


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[.., 2F] (gate columns first) -> [.., F] = silu(gate) * up."""
    _need_cuda(gate_up)
    _bf16(gate_up)
    gate_up = gate_up.contiguous()
    rows, two_f = _rows_cols(gate_up)
    out = torch.empty(*gate_up.shape[:-1], two_f // 2, dtype=torch.bfloat16, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        check(load().b200q_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, two_f // 2, _stream(gate_up)), "b200q_silu_mul")
    return out


def silu_mul_fp8_quantize(gate_up: torch.Tensor):
    """[T, 2F] (gate columns first) -> (FP8 codes [T, F], per-token scales [T]) of silu(gate) * up,
    bit-identical to silu_mul followed by fp8_quantize(.., None)."""
    _need_cuda(gate_up)
    _bf16(gate_up)
    gate_up = gate_up.contiguous()
    rows, two_f = _rows_cols(gate_up)
    codes = torch.empty(*gate_up.shape[:-1], two_f // 2, dtype=torch.uint8, device=gate_up.device)
    scales = torch.empty(rows, dtype=torch.float32, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        check(load().b200q_silu_mul_fp8_quantize(gate_up.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, two_f // 2,
                                                 _stream(gate_up)), "b200q_silu_mul_fp8_quantize")
    return codes, scales


def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _need_cuda(a, b)
    _bf16(a, b)
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty_like(a) if out is None else out
    with torch.cuda.device(a.device):
        check(load().b200q_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream(a)), "b200q_add")
    return out


def expand_heads(src: torch.Tensor, col0: int, heads_out: int, rep: int, head_dim: int) -> torch.Tensor:
    """src [.., W] bf16 -> [.., heads_out*head_dim]: head h is src[.., col0 + (h // rep)*head_dim : +head_dim]."""
    _need_cuda(src)
    _bf16(src)
    src = src.contiguous()
    rows, width = _rows_cols(src)
    out = torch.empty(*src.shape[:-1], heads_out * head_dim, dtype=torch.bfloat16, device=src.device)
    with torch.cuda.device(src.device):
        check(load().b200q_expand_heads(src.data_ptr(), width, col0, out.data_ptr(), rows, heads_out, rep, head_dim, _stream(src)),
              "b200q_expand_heads")
    return out


def expand_heads_fp8_quantize(src: torch.Tensor, col0: int, heads_out: int, rep: int, head_dim: int):
    """`expand_heads` followed by `fp8_quantize(.., None)` in one pass -> (codes [.., heads_out*head_dim], scales [rows]),
    the same bits; the kv slice of a token may hold at most 2048 elements."""
    _need_cuda(src)
    _bf16(src)
    src = src.contiguous()
    rows, width = _rows_cols(src)
    codes = torch.empty(*src.shape[:-1], heads_out * head_dim, dtype=torch.uint8, device=src.device)
    scales = torch.empty(rows, dtype=torch.float32, device=src.device)
    with torch.cuda.device(src.device):
        check(load().b200q_expand_heads_fp8_quantize(src.data_ptr(), width, col0, codes.data_ptr(), scales.data_ptr(), rows, heads_out, rep,
                                                     head_dim, _stream(src)), "b200q_expand_heads_fp8_quantize")
    return codes, scales


def device_status(reset: bool = True) -> int:
    """0, or B200Q_ERR_TIMEOUT (-6) when a GEMM's bounded device-side wait gave up."""
    return load().b200q_device_status(1 if reset else 0)
