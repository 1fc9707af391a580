"""Embedding the b200q ops in Torch-TensorRT engines.

`torch_tensorrt.dynamo.conversion.plugins.custom_op(op_name, capability_validator=None,
priority=STANDARD, supports_dynamic_shapes=False, requires_output_allocator=False)`
(py/torch_tensorrt/dynamo/conversion/plugins/_custom_op.py:13-51) turns a torch.library op
with a fake kernel into a TensorRT quick-deployable plugin plus a converter.  What its
generator can take decides which ops are handed to it:

* only Tensor / float / int / bool / str arguments, anything else raises
  (plugins/_generate_plugin.py:131-158): the ops below have no optional arguments;
* every tensor argument before every scalar argument
  (plugins/_generate_plugin_converter.py:126,143): `quantize_op` satisfies that,
  `dynamic_block_quantize_op(input, block_size, amax, ...)` does not, so a tensors-first alias is
  registered and a hand-written HIGH-priority converter on the original target forwards to it;
* every output descriptor is `tensor_args[0].like()` with the shape the fake kernel computes
  (plugins/_generate_plugin.py:263): the output has the FIRST tensor argument's dtype.  The
  one-node linears `b200_{fp8,nvfp4}_linear[_bias]` take the activation first and return its
  dtype; the GEMMs on raw codes (uint8 in, bf16 out) cannot be described that way and stay
  eager-only.

Neither `torch_tensorrt` nor `tensorrt` ships with this package: when they are missing the
functions report that and return empty lists.
"""
from __future__ import annotations

import logging

import torch

log = logging.getLogger(__name__)

_ALIAS = "tensorrt::b200_dynamic_block_quantize_tensors_first"

# ops the generated plugin + converter can express as they are
PLUGIN_OPS = ("tensorrt::quantize_op", "tensorrt::b200_fp8_linear", "tensorrt::b200_fp8_linear_bias",
              "tensorrt::b200_nvfp4_linear", "tensorrt::b200_nvfp4_linear_bias", _ALIAS)


def _define_tensor_first_alias() -> str:
    try:
        torch.ops.tensorrt.b200_dynamic_block_quantize_tensors_first.default
        return _ALIAS
    except (AttributeError, RuntimeError):
        pass

    @torch.library.custom_op(_ALIAS, mutates_args=())
    def _alias(input: torch.Tensor, amax: torch.Tensor, block_size: int, num_bits: int, exponent_bits: int,
               scale_num_bits: int, scale_exponent_bits: int) -> torch.Tensor:
        return torch.ops.tensorrt.b200_dynamic_block_quantize_op(input, block_size, amax, num_bits, exponent_bits,
                                                                 scale_num_bits, scale_exponent_bits)

    @_alias.register_fake
    def _(input, amax, block_size, num_bits, exponent_bits, scale_num_bits, scale_exponent_bits):
        return torch.empty_like(input)

    return _ALIAS


def make_forwarding_converter(lookup):
    """Converter for `tensorrt::dynamic_block_quantize_op(input, block_size, amax, num_bits,
    exponent_bits, scale_num_bits, scale_exponent_bits)` (argument order:
    py/torch_tensorrt/dynamo/conversion/aten_ops_converters.py:948-960) that moves `amax` in front of
    the scalars and hands the node to the converter generated for the tensors-first alias.
    `lookup(overload)` returns that converter's implementation."""
    alias = torch.ops.tensorrt.b200_dynamic_block_quantize_tensors_first.default
    names = ("input", "block_size", "amax", "num_bits", "exponent_bits", "scale_num_bits", "scale_exponent_bits")

    def dynamic_block_quantize_forward(ctx, target, args, kwargs, name):
        bound = dict(zip(names, args))
        bound.update(kwargs)
        missing = [n for n in names if n not in bound]
        if missing:
            raise ValueError(f"dynamic_block_quantize_op: missing arguments {missing}")
        reordered = (bound["input"], bound["amax"], bound["block_size"], bound["num_bits"], bound["exponent_bits"],
                     bound["scale_num_bits"], bound["scale_exponent_bits"])
        return lookup(alias)(ctx, alias, reordered, {}, name)

    return dynamic_block_quantize_forward


def register_with_torch_tensorrt(custom_op=None, priority=None, converter_decorator=None, lookup=None) -> list[str]:
    """Register the hot-path ops as TensorRT plugins + HIGH-priority converters, and the forwarding
    converter for `dynamic_block_quantize_op`.

    `custom_op`, `priority`, `converter_decorator` (`dynamo_tensorrt_converter`) and `lookup`
    (overload -> registered converter implementation) default to torch_tensorrt's own; tests inject
    fakes.  HIGH matters: STANDARD appends after an existing converter for the same target
    (dynamo/conversion/_ConverterRegistry.py:274-282), so the built-in Q/DQ converters would win.
    Returns the op names registered (the forwarded original last)."""
    if custom_op is None:
        try:
            from torch_tensorrt.dynamo.conversion import plugins
            from torch_tensorrt.dynamo.conversion._ConverterRegistry import (DYNAMO_ATEN_CONVERTERS, ConverterPriority,
                                                                            dynamo_tensorrt_converter)
        except Exception as exc:  # torch_tensorrt / tensorrt absent
            log.warning("torch_tensorrt is not importable (%s); b200q ops stay eager-only", exc)
            return []
        custom_op = plugins.custom_op
        priority = ConverterPriority.HIGH if priority is None else priority
        converter_decorator = converter_decorator or dynamo_tensorrt_converter
        lookup = lookup or (lambda overload: DYNAMO_ATEN_CONVERTERS[overload][0].converter_implementation)
    from .ops import load_ops

    load_ops()
    _define_tensor_first_alias()
    names = list(PLUGIN_OPS)
    for name in names:
        custom_op(name, priority=priority, supports_dynamic_shapes=True)
    if converter_decorator is not None and lookup is not None:
        target = torch.ops.tensorrt.dynamic_block_quantize_op.default
        converter_decorator(target, priority=priority, supports_dynamic_shapes=True)(make_forwarding_converter(lookup))
        names.append("tensorrt::dynamic_block_quantize_op")
    return names
