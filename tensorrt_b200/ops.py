"""Registration of the `tensorrt::` operators.

The quantize ops and the real-quant building blocks live in the C++ shim
(csrc/torch_ops.cpp -> libb200q_torch.so).  The collective op is defined here the way the
reference defines it (py/torch_tensorrt/dynamo/lowering/passes/fuse_distributed_ops.py:57-68:
a torch.library custom op with a fake kernel), unless the reference package already did.
"""
from __future__ import annotations

import torch

from . import _build

_loaded = False


def ops_loaded() -> bool:
    return _loaded


def _define_fused_all_reduce() -> None:
    try:
        torch.ops.tensorrt.fused_nccl_all_reduce.default  # already defined by torch_tensorrt
        return
    except (AttributeError, RuntimeError):
        pass

    @torch.library.custom_op("tensorrt::fused_nccl_all_reduce", mutates_args=())
    def _fused_nccl_all_reduce(inp: torch.Tensor, reduce_op: str, group_name: str) -> torch.Tensor:
        from .tp import all_reduce_by_group_name

        return all_reduce_by_group_name(inp, reduce_op, group_name)

    @_fused_nccl_all_reduce.register_fake
    def _(inp: torch.Tensor, reduce_op: str, group_name: str) -> torch.Tensor:
        return torch.empty_like(inp)


def load_ops() -> None:
    """Build (if needed) and load both native libraries; idempotent."""
    global _loaded
    if _loaded:
        return
    _build.build_cuda()
    shim = _build.build_torch_shim()
    torch.ops.load_library(str(shim))
    _define_fused_all_reduce()
    _loaded = True
