"""Embedding the b200q ops in Torch-TensorRT engines.

`torch_tensorrt.dynamo.conversion.plugins.custom_op(op_name, capability_validator=None,
priority=STANDARD, supports_dynamic_shapes=False, requires_output_allocator=False)`
(py/torch_tensorrt/dynamo/conversion/plugins/_custom_op.py:13-51) turns a torch.library op
with a fake kernel into a TensorRT quick-deployable plugin plus a converter.  Its generated
converter takes every tensor argument before every scalar argument
(plugins/_generate_plugin_converter.py:126,143), which `quantize_op` satisfies and
`dynamic_block_quantize_op(input, block_size, amax, ...)` does not; for the latter a
tensor-first alias is registered and the op itself is routed through it.

Neither `torch_tensorrt` nor `tensorrt` ships with this package: when they are missing the
function reports that and returns the empty list.
"""
from __future__ import annotations

import logging

import torch

log = logging.getLogger(__name__)

# ops whose schema already has tensors first
_DIRECT = ("tensorrt::quantize_op", "tensorrt::b200_fp8_gemm", "tensorrt::b200_nvfp4_gemm")


def _define_tensor_first_alias() -> str:
    name = "tensorrt::b200_dynamic_block_quantize_tensors_first"
    try:
        torch.ops.tensorrt.b200_dynamic_block_quantize_tensors_first.default
        return name
    except (AttributeError, RuntimeError):
        pass

    @torch.library.custom_op(name, mutates_args=())
    def _alias(input: torch.Tensor, amax: torch.Tensor, block_size: int, num_bits: int, exponent_bits: int,
               scale_num_bits: int, scale_exponent_bits: int) -> torch.Tensor:
        return torch.ops.tensorrt.b200_dynamic_block_quantize_op(input, block_size, amax, num_bits, exponent_bits,
                                                                 scale_num_bits, scale_exponent_bits)

    @_alias.register_fake
    def _(input, amax, block_size, num_bits, exponent_bits, scale_num_bits, scale_exponent_bits):
        return torch.empty_like(input)

    return name


def register_with_torch_tensorrt(custom_op=None, priority=None) -> list[str]:
    """Register the hot-path ops as TensorRT plugins + HIGH-priority converters.

    `custom_op` / `priority` default to torch_tensorrt's own
    (`plugins.custom_op`, `ConverterPriority.HIGH`); tests inject fakes.  HIGH matters:
    STANDARD appends after an existing converter for the same target
    (dynamo/conversion/_ConverterRegistry.py:274-282), so the built-in Q/DQ converters would win.
    Returns the op names registered."""
    if custom_op is None:
        try:
            from torch_tensorrt.dynamo.conversion import plugins
            from torch_tensorrt.dynamo.conversion._ConverterRegistry import ConverterPriority
        except Exception as exc:  # torch_tensorrt / tensorrt absent
            log.warning("torch_tensorrt is not importable (%s); b200q ops stay eager-only", exc)
            return []
        custom_op = plugins.custom_op
        priority = ConverterPriority.HIGH if priority is None else priority
    from .ops import load_ops

    load_ops()
    names = list(_DIRECT) + [_define_tensor_first_alias()]
    for name in names:
        custom_op(name, priority=priority, supports_dynamic_shapes=True)
    return names
