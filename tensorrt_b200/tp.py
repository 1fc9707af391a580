"""Tensor-parallel linear stack: column/row sharding and the row-parallel all-reduce.

Sharding follows the reference's manual-slicing export tool
(tools/llm/tensor_parallel_llama_export.py:109-125,151-180): q/k/v/gate/up are column-parallel
(weight rows sliced, no communication), o/down are row-parallel (weight columns sliced, the
partial outputs summed by an all-reduce, bias added once after the reduce).  One process per
GPU; `torch.distributed` (NCCL on GPUs, gloo in CPU tests) carries the collective.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_REDUCE_OPS = {"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.AVG, "min": dist.ReduceOp.MIN,
               "max": dist.ReduceOp.MAX, "product": dist.ReduceOp.PRODUCT}


def resolve_group(group_name: str):
    """Process group registered under `group_name` (the c10d functional-collective name);
    "" or "default" name the world group."""
    if group_name in ("", "default"):
        return dist.group.WORLD
    from torch._C._distributed_c10d import _resolve_process_group

    return _resolve_process_group(group_name)


def all_reduce_by_group_name(inp: torch.Tensor, reduce_op: str, group_name: str) -> torch.Tensor:
    """Eager body of `tensorrt::fused_nccl_all_reduce(inp, reduce_op, group_name)`
    (py/torch_tensorrt/dynamo/lowering/passes/fuse_distributed_ops.py:57-63): out of place,
    identity when the group has a single rank (conversion/impl/nccl_ops.py:409-410)."""
    op = _REDUCE_OPS.get(reduce_op.lower())
    if op is None:
        raise ValueError(f"unsupported reduce_op {reduce_op!r}; expected one of {sorted(_REDUCE_OPS)}")
    if not dist.is_available() or not dist.is_initialized():
        return inp.clone()
    group = resolve_group(group_name)
    if dist.get_world_size(group) == 1:
        return inp.clone()
    out = inp.clone()
    dist.all_reduce(out, op=op, group=group)
    return out


def group_name_of(group=None) -> str:
    group = group or dist.group.WORLD
    return group.group_name


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Column-parallel slice: output features [rank*chunk, (rank+1)*chunk)."""
    if w.shape[0] % world:
        raise ValueError(f"cannot split {w.shape[0]} output features over {world} ranks")
    c = w.shape[0] // world
    return w[rank * c:(rank + 1) * c].contiguous()


def shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Row-parallel slice: input features [rank*chunk, (rank+1)*chunk)."""
    if w.shape[1] % world:
        raise ValueError(f"cannot split {w.shape[1]} input features over {world} ranks")
    c = w.shape[1] // world
    return w[:, rank * c:(rank + 1) * c].contiguous()


class ShapeMismatchError(RuntimeError):
    pass


def check_same_shape(t: torch.Tensor, group=None) -> None:
    """Host-side guard for a collective: every rank contributes (shape, dtype) through an
    object all-gather and raises the same error on all ranks when they differ, instead of
    letting mismatched all-reduce calls hang or corrupt memory on the device."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    mine = (tuple(t.shape), str(t.dtype))
    seen = [None] * dist.get_world_size(group)
    dist.all_gather_object(seen, mine, group=group)
    if any(s != seen[0] for s in seen):
        raise ShapeMismatchError(f"all-reduce operands differ across ranks: {seen}")
