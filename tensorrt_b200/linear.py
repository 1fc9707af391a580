"""Real-quant linear layers: the Q/DQ-wrapped `aten.linear` of the reference, fused.

The reference wraps a linear as `linear(input_quantizer(x), weight_quantizer(W), bias)`
(tools/llm/quantize_utils.py:117-120) and leaves it to TensorRT to fuse the Q/DQ pairs into
an FP8/FP4 GEMM.  Here the weight is quantized once (codes + scales kept on the device),
the activation is quantized by one kernel per call, and one tcgen05 GEMM produces the bf16
output with the dequantization scales and the bias folded into its epilogue.
"""
from __future__ import annotations

import torch
from torch import nn

from . import capi


def fp8_linear(x: torch.Tensor, w_codes: torch.Tensor, w_scales: torch.Tensor, bias=None,
               x_amax: torch.Tensor | None = None) -> torch.Tensor:
    """Per-token (dynamic, or `x_amax` static) FP8 activations x per-channel/per-tensor FP8 weights."""
    x_codes, x_scales = capi.fp8_quantize(x, x_amax)
    return capi.fp8_gemm(x_codes, x_scales, w_codes, w_scales, bias)


def nvfp4_linear(x: torch.Tensor, w_codes, w_scales, w_global, bias=None,
                 x_amax: torch.Tensor | None = None) -> torch.Tensor:
    """NVFP4 W4A4.  `x_amax` is the activation tensor amax (static calibration); None = measured per call."""
    if x_amax is None:
        x_amax = capi.amax(x)
    x_codes, x_scales, x_global = capi.nvfp4_quantize(x, x_amax)
    return capi.nvfp4_gemm(x_codes, x_scales, x_global, w_codes, w_scales, w_global, bias)


class Fp8Linear(nn.Module):
    """y = fp8(x) @ fp8(W)^T + b, weights per-channel (default) or per-tensor E4M3."""

    def __init__(self, w_codes, w_scales, bias=None, input_amax=None):
        super().__init__()
        self.register_buffer("w_codes", w_codes)
        self.register_buffer("w_scales", w_scales)
        self.register_buffer("bias", bias)
        self.register_buffer("input_amax", input_amax)
        self.out_features, self.in_features = w_codes.shape

    @classmethod
    def from_float(cls, linear: nn.Module | torch.Tensor, bias=None, per_channel=True, input_amax=None):
        w = linear.weight if isinstance(linear, nn.Module) else linear
        if isinstance(linear, nn.Module) and bias is None:
            bias = linear.bias
        w = w.detach()
        amax = capi.row_amax(w) if per_channel else capi.amax(w)
        codes, scales = capi.fp8_quantize(w, amax)
        b = None if bias is None else bias.detach().to(torch.bfloat16)
        return cls(codes, scales, b, input_amax)

    def forward(self, x):
        return fp8_linear(x, self.w_codes, self.w_scales, self.bias, self.input_amax)


class Fp8GatedMlp(nn.Module):
    """down(silu(gate(x)) * up(x)) with FP8 linears, the MLP of the decoder models the reference lowers
    (tools/llm: `down_proj(act_fn(gate_proj(x)) * up_proj(x))`, every linear input and weight behind a quantizer).
    The gate and up weights are stacked once ([gate rows; up rows]) so that one GEMM computes both and applies
    the activation in its epilogue; with a static `act_amax` (the calibrated input quantizer of the down
    projection) the epilogue also emits the FP8 codes the down GEMM reads, and a forward is three launches.
    `input_amax` / `act_amax` None = dynamic per-token scales measured by the quantize kernels.  No biases."""

    def __init__(self, gu_codes, gu_scales, down_codes, down_scales, input_amax=None, act_amax=None):
        super().__init__()
        if gu_codes.shape[0] % 256:
            raise ValueError("the intermediate size must be a multiple of 128")
        for name, tensor in (("gu_codes", gu_codes), ("gu_scales", gu_scales), ("down_codes", down_codes), ("down_scales", down_scales),
                             ("input_amax", input_amax), ("act_amax", act_amax)):
            self.register_buffer(name, tensor)

    @classmethod
    def from_float(cls, gate, up, down, per_channel=True, input_amax=None, act_amax=None):
        ws = [(m.weight if isinstance(m, nn.Module) else m).detach() for m in (gate, up, down)]
        if any(isinstance(m, nn.Module) and getattr(m, "bias", None) is not None for m in (gate, up, down)):
            raise ValueError("Fp8GatedMlp has no bias terms")
        if ws[0].shape != ws[1].shape or ws[2].shape != (ws[0].shape[1], ws[0].shape[0]):
            raise ValueError("expected gate, up [F, H] and down [H, F]")
        parts = [capi.fp8_quantize(w, capi.row_amax(w) if per_channel else capi.amax(w)) for w in ws]
        f = ws[0].shape[0]
        # one scale per stacked row (a per-tensor scale is repeated: same products)
        gu_scales = torch.cat([parts[0][1].reshape(-1).expand(f), parts[1][1].reshape(-1).expand(f)])
        return cls(torch.cat([parts[0][0], parts[1][0]]).contiguous(), gu_scales.contiguous(), parts[2][0], parts[2][1], input_amax, act_amax)

    def forward(self, x):
        xq = capi.fp8_quantize(x, self.input_amax)
        tokens = xq[0].numel() // xq[0].shape[-1]
        if tokens >= 256 and self.act_amax is not None and self.act_amax.numel() == 1:
            aq = capi.fp8_gemm_silu_mul_quantize(xq[0], xq[1], self.gu_codes, self.gu_scales, self.act_amax)
        elif tokens >= 256:
            aq = capi.fp8_quantize(capi.fp8_gemm_silu_mul(xq[0], xq[1], self.gu_codes, self.gu_scales), self.act_amax)
        else:   # a decode step: the small-M GEMM and the activation kernels (the same bits)
            gu = capi.fp8_gemm(xq[0], xq[1], self.gu_codes, self.gu_scales)
            aq = capi.fp8_quantize(capi.silu_mul(gu), self.act_amax) if self.act_amax is not None else capi.silu_mul_fp8_quantize(gu)
        return capi.fp8_gemm(aq[0], aq[1], self.down_codes, self.down_scales)


class Nvfp4Linear(nn.Module):
    """y = nvfp4(x) @ nvfp4(W)^T + b (block 16, E4M3 block scales, fp32 global scales)."""

    def __init__(self, w_codes, w_scales, w_global, bias=None, input_amax=None):
        super().__init__()
        self.register_buffer("w_codes", w_codes)
        self.register_buffer("w_scales", w_scales)
        self.register_buffer("w_global", w_global)
        self.register_buffer("bias", bias)
        self.register_buffer("input_amax", input_amax)
        self.out_features, self.in_features = w_codes.shape[0], w_codes.shape[1] * 2

    @classmethod
    def from_float(cls, linear: nn.Module | torch.Tensor, bias=None, input_amax=None):
        w = linear.weight if isinstance(linear, nn.Module) else linear
        if isinstance(linear, nn.Module) and bias is None:
            bias = linear.bias
        w = w.detach()
        codes, scales, g = capi.nvfp4_quantize(w, capi.amax(w))
        b = None if bias is None else bias.detach().to(torch.bfloat16)
        return cls(codes, scales, g, b, input_amax)

    def forward(self, x):
        return nvfp4_linear(x, self.w_codes, self.w_scales, self.w_global, self.bias, self.input_amax)


class QuantizedLinear(nn.Module):
    """Eager Q/DQ linear with the reference's structure (tools/llm/quantize_utils.py:87-120):
    both quantizers are the fake-quant `tensorrt::` ops, the matmul runs in the input dtype.
    Used to check the fused layers against the unfused graph TensorRT would be given."""

    def __init__(self, weight, bias=None, mode="fp8", input_amax=None, weight_amax=None):
        super().__init__()
        if mode not in ("fp8", "nvfp4"):
            raise ValueError(f"mode must be 'fp8' or 'nvfp4', got {mode!r}")
        self.mode = mode
        self.register_buffer("weight", weight)
        self.register_buffer("bias", bias)
        self.register_buffer("input_amax", input_amax)
        self.register_buffer("weight_amax", weight_amax if weight_amax is not None else capi.amax(weight))

    def _q(self, t, amax):
        if self.mode == "fp8":
            return torch.ops.tensorrt.quantize_op(t, amax, 8, 4, False, False)
        return torch.ops.tensorrt.dynamic_block_quantize_op(t, 16, amax, 4, 2, 8, 4)

    def forward(self, x):
        xa = self.input_amax if self.input_amax is not None else capi.amax(x)
        return torch.nn.functional.linear(self._q(x, xa), self._q(self.weight, self.weight_amax), self.bias)
