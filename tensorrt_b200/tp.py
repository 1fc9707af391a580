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


def probe_group_names(backend: str | None = "nccl", limit: int = 20) -> list[str]:
    """Names among "0" .. str(limit - 1) that resolve to a registered process group (of `backend`
    when given).  The reference's runtime resolves an engine's group this way when none was pinned
    (core/runtime/TRTEngine.cpp:845-857): gaps in the numbering are skipped, and the result is only
    usable when exactly one group is found."""
    from torch._C._distributed_c10d import _resolve_process_group

    found = []
    for i in range(limit):
        try:
            group = _resolve_process_group(str(i))
        except Exception:  # unknown name: a gap in the numbering
            continue
        if group is None:
            continue
        if backend is None or dist.get_backend(group) == backend:
            found.append(str(i))
    return found


def auto_group_name(backend: str | None = "nccl") -> str:
    """The single registered group's name; raises when there is none or more than one (a TP + DP
    job must pin the group explicitly, as in the reference)."""
    names = probe_group_names(backend)
    if len(names) != 1:
        raise RuntimeError(f"cannot pick a process group automatically: found {names or 'none'}; pass the group name")
    return names[0]


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


def replicate_row_parallel_bias(bias, group=None, device=None):
    """Bias of a row-parallel linear in the form the fused peer-memory path needs.

    Two conventions meet here.  "Linear, then all-reduce" (the reference's _RowParallelLinear,
    tools/llm/tensor_parallel_llama_export.py:109-125) sums whatever every rank adds, so the
    checkpoint loader keeps a row-parallel bias on rank 0 only (checkpoint.load_quantized_linears).
    The fused path (FusedRowParallel, b200q_reduce_gather and its siblings) adds the bias AFTER the
    sum, on the rank that owns each row, so every rank must hold the full bias.  This collective
    call converts the first form into the second: rank 0's bias is broadcast to all ranks; returns
    None on every rank when rank 0 has none.  A rank other than 0 that holds a bias of its own is an
    error (it would have been summed twice by the unfused path)."""
    group = group or dist.group.WORLD
    world = dist.get_world_size(group)
    if world == 1:
        return bias
    rank = dist.get_rank(group)
    have = [None] * world
    dist.all_gather_object(have, None if bias is None else (tuple(bias.shape), str(bias.dtype)), group=group)
    if have[0] is None:
        if any(h is not None for h in have[1:]):
            raise ValueError(f"a row-parallel bias must live on rank 0 (and optionally, identically, on every rank), got {have}")
        return None
    if any(h is not None and h != have[0] for h in have[1:]):
        raise ValueError(f"row-parallel bias differs across ranks: {have}")
    if all(h == have[0] for h in have):
        return bias                                       # already replicated
    shape, dtype = have[0]
    if bias is None:
        bias = torch.empty(shape, dtype=getattr(torch, dtype.split(".")[-1]), device=device or "cpu")
    src = dist.get_global_rank(group, 0) if group is not dist.group.WORLD else 0
    dist.broadcast(bias, src=src, group=group)
    return bias


class CommContext:
    """The library's own communication context (include/b200q.h: b200q_comm_*): symmetric device buffers
    whose peer mappings come from CUDA IPC, exchanged through an all-gather the host supplies.  This
    wrapper supplies `torch.distributed.all_gather_object` on `group` (any backend; gloo works) as that
    all-gather; a C or C++ host passes its own.  `alloc(nbytes)` is collective and returns the list of
    `world` device pointers valid in this process plus a uint8 tensor view of the local buffer."""

    def __init__(self, group=None):
        import ctypes

        from . import _lib

        self.group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        lib = _lib.load()

        def allgather(user, send, recv, nbytes):
            try:
                mine = ctypes.string_at(send, nbytes)
                parts = [None] * self.world
                dist.all_gather_object(parts, mine, group=self.group)
                ctypes.memmove(recv, b"".join(parts), nbytes * self.world)
                return 0
            except Exception:  # reported as a status code: nothing may propagate through the C caller
                return 1

        self._cb = _lib.ALLGATHER_FN(allgather)          # kept alive as long as the context
        handle = ctypes.c_void_p()
        _lib.check(lib.b200q_comm_create(self.rank, self.world, self._cb, None, ctypes.byref(handle)), "b200q_comm_create")
        self._handle, self._lib = handle, lib

    def alloc(self, nbytes: int):
        import ctypes

        from . import _lib

        ptrs = (ctypes.c_void_p * 8)()
        _lib.check(self._lib.b200q_comm_alloc(self._handle, nbytes, ptrs), "b200q_comm_alloc")
        addrs = [int(ptrs[r]) for r in range(self.world)]
        return addrs, _device_view(addrs[self.rank], nbytes)

    def close(self) -> None:
        if self._handle is not None:
            from . import _lib

            _lib.check(self._lib.b200q_comm_destroy(self._handle), "b200q_comm_destroy")
            self._handle = None


def _device_view(ptr: int, nbytes: int) -> torch.Tensor:
    """uint8 tensor over `nbytes` of device memory at `ptr` (memory owned by someone else)."""
    class _Raw:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}

    return torch.as_tensor(_Raw(), device=torch.device("cuda", torch.cuda.current_device()))


def _symmetric_buffers(sizes, group, comm: "CommContext | None"):
    """For every size a zeroed uint8 buffer on each rank plus its `world` peer pointers: through the
    library's own context when one is given, else through torch's symmetric-memory allocator."""
    if comm is not None:
        out = []
        for size in sizes:
            addrs, local = comm.alloc(size)
            out.append((local, addrs))
        return out
    import torch.distributed._symmetric_memory as symm_mem

    dev = torch.device("cuda", torch.cuda.current_device())
    out = []
    for size in sizes:
        t = symm_mem.empty(size, dtype=torch.uint8, device=dev)
        t.zero_()
        h = symm_mem.rendezvous(t, group.group_name)
        out.append((t, [int(p) for p in h.buffer_ptrs], h))
    return out


class FusedRowParallel:
    """Row-parallel quantized linear + all-reduce as two b200q launches over peer memory
    (include/b200q.h: b200q_*_gemm_reduce_scatter, b200q_reduce_gather) instead of a GEMM followed
    by an NCCL all-reduce.  torch's symmetric-memory allocator provides the peer mappings (one
    rendezvous at construction); nothing else of it is used: the data path and the flag
    protocol are this library's own kernels.

    `max_rows` x `n_out` bf16 bounds the buffers.  Calls whose row count is not a multiple of
    world * 128 (decode steps) fall back to `fallback(x, qw, amax)`, the NCCL path.
    The returned tensor is a view of this rank's output buffer and is valid until the next call.

    Bias convention: `bias` arguments are added once, after the sum, by the rank that owns each
    row, so EVERY rank passes the same full bias (or every rank passes None).  A checkpoint-loaded
    row-parallel linear keeps its bias on rank 0 only; convert it once with
    `replicate_row_parallel_bias`.  The first use of a bias tensor is checked across ranks.
    """

    def __init__(self, mode: str, max_rows: int, n_out: int, group=None, fallback=None, sharded: bool = False, comm=None):
        """`sharded`: also allocate the gathered-activation buffers of the token-sharded residual
        stream (`partials_to_owners` / `reduce_norm_quantize` / `reduce_add`).  `comm`: a `CommContext`
        to take the peer buffers from (the library's own CUDA-IPC context) instead of torch's
        symmetric-memory allocator."""
        import os

        # plain peer mappings are all this path needs; keep the allocator from also binding the
        # buffers to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.mode, self.group, self.fallback = mode, group or dist.group.WORLD, fallback
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("FusedRowParallel supports at most 8 ranks")
        self.max_rows, self.n_out, self.sharded, self.comm = max_rows, n_out, sharded, comm
        # one set of peer buffers, flags and epoch counter per CUDA stream that calls in: calls on
        # different streams may overlap on the device and must not share them
        self._ctx: dict = {}
        self._bias_seen: set = set()

    def prepare(self, rows: int, streams=None) -> None:
        """Allocate the peer buffers for calls of up to `rows` rows on each of `streams` (default:
        the current stream) now.  Collective: every rank calls it with the same arguments.  Doing
        this before a timed region or a stream capture keeps the allocation, the rendezvous and
        the barrier they need out of the first forward."""
        for st in (streams or [torch.cuda.current_stream()]):
            with torch.cuda.stream(st):
                self._context(rows)

    def _checked_bias(self, bias):
        """bf16 contiguous bias, or None; the first time a tensor is seen its presence and shape are
        compared across ranks (a bias on some ranks only would silently bias some rows only)."""
        if bias is not None:
            bias = bias.to(torch.bfloat16).contiguous()
        key = None if bias is None else (bias.data_ptr(), tuple(bias.shape))
        if key not in self._bias_seen:
            have = [None] * self.world
            dist.all_gather_object(have, None if bias is None else tuple(bias.shape), group=self.group)
            if any(h != have[0] for h in have):
                raise ValueError(f"the fused row-parallel path needs the same full bias on every rank, got {have}; "
                                 "see tp.replicate_row_parallel_bias")
            self._bias_seen.add(key)
        return bias

    def _context(self, rows: int):
        """Buffers of the calling stream, (re)allocated collectively: every rank reaches this point
        with the same stream order and the same `rows`."""
        import ctypes

        from . import _lib

        key = torch.cuda.current_stream().cuda_stream
        ctx = self._ctx.get(key)
        if ctx is not None and ctx["rows"] >= rows:
            return ctx
        nbytes = rows * self.n_out * 2
        sizes = [nbytes, nbytes, 4096]
        if self.sharded:
            sizes += [rows * self.n_out, rows * 4]           # gathered FP8 codes and per-token scales
        bufs = _symmetric_buffers(sizes, self.group, self.comm)
        ptrs = [b[1] for b in bufs]
        torch.cuda.current_stream().synchronize()
        dist.barrier(self.group)
        peers = _lib.Peers()
        peers.rank, peers.world = self.rank, self.world
        for r in range(self.world):
            peers.recv[r], peers.out[r], peers.flags[r] = ptrs[0][r], ptrs[1][r], ptrs[2][r]
        ctx = {"rows": rows, "bufs": bufs, "peers": peers, "ref": ctypes.byref(peers), "out": bufs[1][0], "epoch": 0}
        if self.sharded:
            gp = _lib.GatherPeers()
            gp.rank, gp.world = self.rank, self.world
            for r in range(self.world):
                gp.recv[r], gp.flags[r], gp.codes[r], gp.scales[r] = ptrs[0][r], ptrs[2][r], ptrs[3][r], ptrs[4][r]
            ctx.update(gather=gp, gather_ref=ctypes.byref(gp), codes=bufs[3][0], scales=bufs[4][0])
        self._ctx[key] = ctx
        return ctx

    def __call__(self, x, qw, amax=None, bias=None) -> torch.Tensor:
        """`x`: bf16 activation [rows, K/world] or an already quantized operand (FP8: (codes,
        per-token scales))."""
        from ._lib import check, load

        rows = x[0].shape[0] if isinstance(x, tuple) else x.shape[0]
        n = self.n_out
        if rows % (self.world * 128) or rows > self.max_rows:
            if self.fallback is None:
                raise ValueError(f"{rows} rows: need a multiple of {self.world * 128} and at most {self.max_rows}")
            return self.fallback(x, qw, amax)
        b = self._checked_bias(bias)
        ctx = self._gemm_to_owners(x, qw, amax)
        lib = load()
        check(lib.b200q_reduce_gather(ctx["ref"], None if b is None else b.data_ptr(), rows, n, ctx["epoch"],
                                      torch.cuda.current_stream().cuda_stream, None), "b200q_reduce_gather")
        return ctx["out"][: rows * n * 2].view(torch.bfloat16).view(rows, n)

    def _gemm_to_owners(self, x, qw, amax=None):
        """Quantize x, run the GEMM whose epilogue stores every partial tile into the receive buffer
        of the rank owning those rows; opens a new epoch.  Returns the calling stream's context."""
        from . import capi
        from ._lib import check, load

        rows, n = (x[0].shape[0] if isinstance(x, tuple) else x.shape[0]), self.n_out
        lib = load()
        ctx = self._context(rows)
        ref = ctx["ref"]
        stream = torch.cuda.current_stream().cuda_stream
        if self.mode == "fp8":
            xc, xs = x if isinstance(x, tuple) else capi.fp8_quantize(x, None)
            k = xc.shape[1]
            check(lib.b200q_fp8_gemm_reduce_scatter(xc.data_ptr(), xs.data_ptr(), xs.numel(), qw[0].data_ptr(), qw[1].data_ptr(),
                                                    qw[1].numel(), ref, rows, n, k, stream, None), "b200q_fp8_gemm_reduce_scatter")
        else:
            xc, xs, xg = x if isinstance(x, tuple) else capi.nvfp4_quantize(x, capi.amax(x) if amax is None else amax)
            k = xc.shape[1] * 2
            check(lib.b200q_nvfp4_gemm_reduce_scatter(xc.data_ptr(), xs.data_ptr(), xg.data_ptr(), qw[0].data_ptr(), qw[1].data_ptr(),
                                                      qw[2].data_ptr(), ref, rows, n, k, stream, None),
                  "b200q_nvfp4_gemm_reduce_scatter")
        ctx["epoch"] += 1
        ctx["pending_rows"] = rows
        return ctx

    # ---- token-sharded residual stream -------------------------------------------------
    def usable(self, rows: int) -> bool:
        return rows % (self.world * 128) == 0 and rows <= self.max_rows

    def partials_to_owners(self, x, qw, amax=None) -> None:
        """First half of a row-parallel linear: the partial outputs land at their owners; one of
        `reduce_norm_quantize` / `reduce_add` must follow on the same stream."""
        rows = x[0].shape[0] if isinstance(x, tuple) else x.shape[0]
        if not self.usable(rows):
            raise ValueError(f"{rows} rows: need a multiple of {self.world * 128} and at most {self.max_rows}")
        self._gemm_to_owners(x, qw, amax)

    def reduce_norm_quantize(self, h_shard: torch.Tensor, norm_weight: torch.Tensor, eps: float, bias=None):
        """Second half, fused with the start of the next layer: h_shard (this rank's residual rows,
        updated in place) += reduced partials; returns the FP8 codes [rows, n] and per-token scales
        [rows] of rms_norm(h) for ALL tokens (views of this rank's gathered buffers, valid until
        the next call on this stream)."""
        from ._lib import check, load

        ctx = self._ctx[torch.cuda.current_stream().cuda_stream]
        rows, n = ctx.pop("pending_rows"), self.n_out
        if tuple(h_shard.shape) != (rows // self.world, n) or not h_shard.is_contiguous() or h_shard.dtype != torch.bfloat16:
            raise ValueError(f"h_shard must be a contiguous bf16 [{rows // self.world}, {n}] tensor")
        b = self._checked_bias(bias)
        w = norm_weight.to(torch.bfloat16).contiguous()
        check(load().b200q_reduce_add_rms_norm_fp8_quantize_gather(
            ctx["gather_ref"], None if b is None else b.data_ptr(), h_shard.data_ptr(), w.data_ptr(), float(eps), rows, n,
            ctx["epoch"], torch.cuda.current_stream().cuda_stream, None), "b200q_reduce_add_rms_norm_fp8_quantize_gather")
        return ctx["codes"][: rows * n].view(rows, n), ctx["scales"][: rows * 4].view(torch.float32)

    def reduce_add(self, h_shard: torch.Tensor, bias=None) -> torch.Tensor:
        """Second half at the end of a stack: the full [rows, n] bf16 result h + reduced partials on
        every rank (a view of this rank's output buffer, valid until the next call)."""
        from ._lib import check, load

        ctx = self._ctx[torch.cuda.current_stream().cuda_stream]
        rows, n = ctx.pop("pending_rows"), self.n_out
        if tuple(h_shard.shape) != (rows // self.world, n) or not h_shard.is_contiguous() or h_shard.dtype != torch.bfloat16:
            raise ValueError(f"h_shard must be a contiguous bf16 [{rows // self.world}, {n}] tensor")
        b = self._checked_bias(bias)
        check(load().b200q_reduce_add_gather(ctx["ref"], None if b is None else b.data_ptr(), h_shard.data_ptr(), rows, n,
                                             ctx["epoch"], torch.cuda.current_stream().cuda_stream, None), "b200q_reduce_add_gather")
        return ctx["out"][: rows * n * 2].view(torch.bfloat16).view(rows, n)


class PullRowParallel:
    """Row-parallel quantized linear + all-reduce for a handful of tokens (decode steps), with the
    following residual add, RMSNorm and FP8 quantize fused in: the GEMM writes this rank's partial into
    its own symmetric buffer, one tiny launch signals the peers, and every rank's reduction kernel
    pulls all partials over peer memory (include/b200q.h: b200q_pull_signal, b200q_pull_reduce_*).  No
    collective-library call is involved and the call counter lives on the device, so a whole decode
    step can be captured in a CUDA graph and replayed.

    Same method names as the token-sharded part of `FusedRowParallel` (`partials_to_owners`,
    `reduce_norm_quantize`, `reduce_add`), but the residual stream `h` is the full replicated [rows, n]
    tensor here.  Two partial buffers alternate between consecutive calls; a captured step must hold an
    even number of all-reduces so that replays start on the same buffer (a decoder layer has two)."""

    def __init__(self, mode: str, max_rows: int, n_out: int, group=None, comm=None):
        import ctypes
        import os

        from . import _lib

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        if max_rows > 1024:
            raise ValueError("PullRowParallel serves at most 1024 rows per call")
        self.mode, self.group = mode, group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("PullRowParallel supports at most 8 ranks")
        self.max_rows, self.n_out = max_rows, n_out
        nbytes = max_rows * n_out * 2
        self._bufs = _symmetric_buffers([4096, nbytes, nbytes], self.group, comm)
        self._peers, self._refs, self._partial = [], [], []
        flag_ptrs = self._bufs[0][1]
        for local, ptrs, *_ in self._bufs[1:]:
            peers = _lib.PullPeers()
            peers.rank, peers.world = self.rank, self.world
            for r in range(self.world):
                peers.partial[r], peers.flags[r] = ptrs[r], flag_ptrs[r]
            self._peers.append(peers)
            self._refs.append(ctypes.byref(peers))
            self._partial.append(local.view(torch.bfloat16))
        torch.cuda.current_stream().synchronize()
        dist.barrier(self.group)
        self._slot = 0
        self._pending = None
        self._bias_seen: set = set()

    _checked_bias = FusedRowParallel._checked_bias

    def usable(self, rows: int) -> bool:
        return 0 < rows <= self.max_rows

    def partials_to_owners(self, x, qw, amax=None) -> None:
        """The GEMM of a row-parallel linear into this rank's partial buffer, then the signal."""
        from . import capi
        from ._lib import check, load

        rows = x[0].shape[0] if isinstance(x, tuple) else x.shape[0]
        if not self.usable(rows):
            raise ValueError(f"{rows} rows: at most {self.max_rows}")
        slot = self._slot
        out = self._partial[slot][: rows * self.n_out].view(rows, self.n_out)
        if self.mode == "fp8":
            xc, xs = x if isinstance(x, tuple) else capi.fp8_quantize(x, None)
            capi.fp8_gemm(xc, xs, qw[0], qw[1], None, out=out)
        else:
            xc, xs, xg = x if isinstance(x, tuple) else capi.nvfp4_quantize(x, capi.amax(x) if amax is None else amax)
            capi.nvfp4_gemm(xc, xs, xg, qw[0], qw[1], qw[2], None, out=out)
        check(load().b200q_pull_signal(self._refs[slot], torch.cuda.current_stream().cuda_stream), "b200q_pull_signal")
        self._pending = (slot, rows)
        self._slot = slot ^ 1

    def _take_pending(self, h: torch.Tensor):
        if self._pending is None:
            raise RuntimeError("no row-parallel GEMM is pending: call partials_to_owners first")
        slot, rows = self._pending
        self._pending = None
        if tuple(h.shape) != (rows, self.n_out) or not h.is_contiguous() or h.dtype != torch.bfloat16:
            raise ValueError(f"h must be a contiguous bf16 [{rows}, {self.n_out}] tensor")
        return slot, rows

    def reduce_norm_quantize(self, h: torch.Tensor, norm_weight: torch.Tensor, eps: float, bias=None):
        """h (full residual rows, updated in place) += sum of all ranks' partials (+ bias); returns the
        FP8 codes [rows, n] and per-token scales [rows] of rms_norm(h)."""
        from ._lib import check, load

        slot, rows = self._take_pending(h)
        b = self._checked_bias(bias)
        w = norm_weight.to(torch.bfloat16).contiguous()
        codes = torch.empty(rows, self.n_out, dtype=torch.uint8, device=h.device)
        scales = torch.empty(rows, dtype=torch.float32, device=h.device)
        check(load().b200q_pull_reduce_add_rms_norm_fp8_quantize(
            self._refs[slot], None if b is None else b.data_ptr(), h.data_ptr(), w.data_ptr(), float(eps), codes.data_ptr(),
            scales.data_ptr(), rows, self.n_out, torch.cuda.current_stream().cuda_stream, None),
            "b200q_pull_reduce_add_rms_norm_fp8_quantize")
        return codes, scales

    def reduce_add(self, h: torch.Tensor, bias=None) -> torch.Tensor:
        """End of a stack: h += sum of all ranks' partials (+ bias), in place; returns h."""
        from ._lib import check, load

        slot, rows = self._take_pending(h)
        b = self._checked_bias(bias)
        check(load().b200q_pull_reduce_add(self._refs[slot], None if b is None else b.data_ptr(), h.data_ptr(), rows, self.n_out,
                                           torch.cuda.current_stream().cuda_stream, None), "b200q_pull_reduce_add")
        return h
