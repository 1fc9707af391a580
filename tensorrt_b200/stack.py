"""Llama-shaped decoder *linear* stack with quantized linears, optionally tensor-parallel.

One layer:  h -> RMSNorm -> QKV linear -> "attention" (identity on the V slice, every kv head
repeated n_q/n_kv times up to the query width) -> O linear -> (all-reduce) -> residual ->
RMSNorm -> gate/up linear -> silu(gate) * up -> down linear -> (all-reduce) -> residual.

Tensor parallelism follows the reference's plan (tools/llm/tensor_parallel_llama_llm.py:134-157;
manual-slicing twin tools/llm/tensor_parallel_llama_export.py:109-190): q/k/v/gate/up are
column-parallel (weight rows sliced, no communication), o/down row-parallel (weight columns
sliced, partial outputs summed by `tensorrt::fused_nccl_all_reduce` semantics).  Each rank
quantizes the activation slice it owns (per-token amax over the local slice for FP8, a
tensor amax of the local slice for NVFP4).

With `forward(.., sharded=True)` the residual stream itself is sharded by tokens (sequence-parallel form of
the same plan): a row-parallel linear ends in a reduce-scatter instead of an all-reduce, the
residual add + RMSNorm + quantize run on the T/W tokens a rank owns, and the column-parallel
linear that follows starts with an all-gather of the *quantized* activations (1 byte per element
plus one scale per token instead of 2 bytes).  Same arithmetic per token, half the bytes on
NVLink and no replicated norm work.

The numerical work is done by a `backend` object.  `CudaBackend` (the product) calls the b200q
kernels through the C ABI; tests drive the same layer logic on CPU/gloo ranks with a backend
built from the CPU oracle.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import capi


@dataclass(frozen=True)
class StackConfig:
    hidden: int
    n_q: int
    n_kv: int
    head_dim: int
    ffn: int
    layers: int
    mode: str = "fp8"          # "fp8" (per-token activations x per-channel weights) or "nvfp4" (W4A4)
    eps: float = 1e-5
    # attention core between the QKV and O linears: "identity" = the V slice with every kv head repeated to the
    # query width (the linear-stack stand-in); "fp8_sdpa" = causal FP8 attention (Q, K, V quantized per tensor,
    # softmax output quantized at scale 1/448) over sequences of `seq_len` tokens, tokens sequence-major
    attention: str = "identity"
    seq_len: int = 0

    @property
    def q_width(self):
        return self.n_q * self.head_dim

    @property
    def kv_width(self):
        return self.n_kv * self.head_dim

    def check(self, world: int = 1):
        if self.mode not in ("fp8", "nvfp4"):
            raise ValueError(f"mode must be 'fp8' or 'nvfp4', got {self.mode!r}")
        if self.n_q % self.n_kv:
            raise ValueError("n_q must be a multiple of n_kv")
        if self.attention not in ("identity", "fp8_sdpa"):
            raise ValueError(f"attention must be 'identity' or 'fp8_sdpa', got {self.attention!r}")
        if self.attention == "fp8_sdpa" and (self.seq_len <= 0 or self.head_dim % 16 or self.head_dim > 128):
            raise ValueError("attention='fp8_sdpa' needs seq_len > 0 and a head dimension that is a multiple of 16 up to 128")
        if self.n_q % world or self.n_kv % world or self.ffn % world:
            raise ValueError(f"heads ({self.n_q}/{self.n_kv}) and ffn ({self.ffn}) must divide by the TP size {world}")

    def weights_per_layer(self):
        return self.hidden * (self.q_width + 2 * self.kv_width) + self.hidden * self.q_width + 3 * self.hidden * self.ffn

    def flops_per_token(self):
        return 2 * self.weights_per_layer() * self.layers


LLAMA3_8B = StackConfig(hidden=4096, n_q=32, n_kv=8, head_dim=128, ffn=14336, layers=32, mode="nvfp4")
LLAMA3_70B = StackConfig(hidden=8192, n_q=64, n_kv=8, head_dim=128, ffn=28672, layers=80, mode="fp8")


# ----------------------------------------------------------------------------- sharding
def shard_layer_weights(layer: dict, cfg: StackConfig, rank: int, world: int) -> dict:
    """Full-precision layer weights -> this rank's slices.  `wqkv` rows are
    [q heads | k heads | v heads], `wgu` rows are [gate | up]."""
    q, kv = cfg.q_width, cfg.kv_width
    qs, kvs, fs = q // world, kv // world, cfg.ffn // world
    wq, wk, wv = layer["wqkv"][:q], layer["wqkv"][q:q + kv], layer["wqkv"][q + kv:]
    gate, up = layer["wgu"][:cfg.ffn], layer["wgu"][cfg.ffn:]
    return {
        "norm1": layer["norm1"], "norm2": layer["norm2"],
        "wqkv": torch.cat([wq[rank * qs:(rank + 1) * qs], wk[rank * kvs:(rank + 1) * kvs], wv[rank * kvs:(rank + 1) * kvs]]).contiguous(),
        "wo": layer["wo"][:, rank * qs:(rank + 1) * qs].contiguous(),
        "wgu": torch.cat([gate[rank * fs:(rank + 1) * fs], up[rank * fs:(rank + 1) * fs]]).contiguous(),
        "wdown": layer["wdown"][:, rank * fs:(rank + 1) * fs].contiguous(),
    }


# ----------------------------------------------------------------------------- backends
class CudaBackend:
    """b200q kernels through the C ABI."""

    def __init__(self, mode: str, fuse_gate_up: bool = True):
        """`fuse_gate_up` False keeps silu(gate) * up in its own kernel after the gate/up GEMM (A/B measurements)."""
        self.mode, self.fuse_gate_up = mode, fuse_gate_up

    def prepare_weight(self, w: torch.Tensor):
        if self.mode == "fp8":
            return capi.fp8_quantize(w, capi.row_amax(w))
        return capi.nvfp4_quantize(w, capi.amax(w))

    def quantize(self, x: torch.Tensor, amax: torch.Tensor | None = None):
        """Activation -> quantized operand of `matmul`.  `amax`: calibrated (static) tensor amax for
        NVFP4, None = measured on this input; FP8 activations are scaled per token in the kernel."""
        if self.mode == "fp8":
            return capi.fp8_quantize(x, None)
        return capi.nvfp4_quantize(x, capi.amax(x) if amax is None else amax)

    def matmul(self, xq, qw) -> torch.Tensor:
        if self.mode == "fp8":
            return capi.fp8_gemm(xq[0], xq[1], qw[0], qw[1], None)
        return capi.nvfp4_gemm(xq[0], xq[1], xq[2], qw[0], qw[1], qw[2], None)

    def linear(self, x, qw, amax: torch.Tensor | None = None) -> torch.Tensor:
        """`x`: bf16 activation, or an already quantized operand (tuple, as `quantize` returns)."""
        return self.matmul(x if isinstance(x, tuple) else self.quantize(x, amax), qw)

    def gate_up_activation(self, xq, qw):
        """Quantized input of the down projection straight from the gate/up GEMM: silu(gate) * up is applied
        in the GEMM's epilogue (the [T, 2F] bf16 tensor is never written), then quantized per token.  FP8 with
        at least 256 tokens and F a multiple of 128; None otherwise (the caller takes the unfused kernels)."""
        if not self.fuse_gate_up or self.mode != "fp8" or xq[0].shape[0] < 256 or qw[0].shape[0] % 256:
            return None
        return capi.fp8_quantize(capi.fp8_gemm_silu_mul(xq[0], xq[1], qw[0], qw[1], None), None)

    def expand_heads_quantize(self, src, col0, heads_out, rep, head_dim):
        """The repeated-head stand-in for attention together with the per-token quantize in front of the O
        projection (FP8; the kv slice of a token must fit one warp's registers), else None."""
        if self.mode != "fp8" or (heads_out // rep) * head_dim > 2048:
            return None
        return capi.expand_heads_fp8_quantize(src, col0, heads_out, rep, head_dim)

    def silu_mul_quantize(self, gate_up: torch.Tensor):
        """silu(gate) * up as the quantized operand of the down projection (one kernel), or None
        when the mode has no fused form (NVFP4 block quantize needs the tensor amax first)."""
        if self.mode != "fp8":
            return None
        return capi.silu_mul_fp8_quantize(gate_up)

    def add_norm_quantize(self, h: torch.Tensor, delta, weight: torch.Tensor, eps: float, amax=None):
        """(h + delta, quantized rms_norm(h + delta)).  FP8: one fused kernel; NVFP4: add, norm and
        block quantize as separate kernels (the block quantize needs the tensor amax)."""
        if self.mode == "fp8":
            h_new, codes, scales = capi.add_rms_norm_fp8_quantize(h, delta, weight, eps)
            return h_new, (codes, scales)
        h_new = h if delta is None else capi.add(h, delta)
        x = capi.rms_norm(h_new, weight, eps)
        return h_new, self.quantize(x, amax)

    def causal_attention(self, qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, seq_len: int) -> torch.Tensor:
        """qkv [tokens, (n_q + 2 n_kv) * head_dim] of whole sequences -> causal FP8 attention output
        [tokens, n_q * head_dim]; Q, K, V quantized per tensor at their measured abs-max."""
        t = qkv.shape[0]
        if seq_len <= 0 or t % seq_len:
            raise ValueError(f"{t} tokens are not whole sequences of {seq_len}")
        b, qw, kvw = t // seq_len, n_q * head_dim, n_kv * head_dim
        heads = lambda x, n: x.reshape(b, seq_len, n, head_dim).permute(0, 2, 1, 3).contiguous()  # noqa: E731
        q, k, v = heads(qkv[:, :qw], n_q), heads(qkv[:, qw:qw + kvw], n_kv), heads(qkv[:, qw + kvw:], n_kv)
        out = capi.fp8_sdpa(q, k, v, capi.amax(q), capi.amax(k), capi.amax(v), True)
        return out.permute(0, 2, 1, 3).reshape(t, qw)

    def measure_norm_amax(self, h, delta, weight, eps):
        if self.mode != "nvfp4":
            return None
        h_new = h if delta is None else capi.add(h, delta)
        return capi.amax(capi.rms_norm(h_new, weight, eps))

    def measure_amax(self, x: torch.Tensor):
        return capi.amax(x) if self.mode == "nvfp4" else None

    rms_norm = staticmethod(capi.rms_norm)
    silu_mul = staticmethod(capi.silu_mul)
    add = staticmethod(capi.add)
    expand_heads = staticmethod(capi.expand_heads)


# ----------------------------------------------------------------------------- collectives
class AllReduce:
    """Row-parallel sum over the TP group; `slabs` > 1 splits the rows so that the collective of
    one slab overlaps the caller's work on the next (the caller passes a generator of slabs)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t


class ShardedComm:
    """Collectives of the token-sharded residual stream: reduce-scatter of row-parallel partial
    outputs and all-gather of quantized activations, both along the token axis.  NCCL runs the
    native collectives; gloo (CPU tests) has no reduce-scatter, so it reduces and slices."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.native = dist.get_backend(group) == "nccl"

    def shard(self, t: torch.Tensor) -> torch.Tensor:
        rows = t.shape[0] // self.world
        return t[self.rank * rows:(self.rank + 1) * rows]

    def reduce_scatter(self, part: torch.Tensor) -> torch.Tensor:
        if part.shape[0] % self.world:
            raise ValueError(f"{part.shape[0]} tokens do not divide over {self.world} ranks")
        if self.native:
            out = part.new_empty((part.shape[0] // self.world,) + tuple(part.shape[1:]))
            dist.reduce_scatter_tensor(out, part, op=dist.ReduceOp.SUM, group=self.group)
            return out
        dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
        return self.shard(part).contiguous()

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        if self.native:
            out = t.new_empty((t.shape[0] * self.world,) + tuple(t.shape[1:]))
            dist.all_gather_into_tensor(out, t, group=self.group)
            return out
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t, group=self.group)
        return torch.cat(parts, dim=0)

    def all_gather_quantized(self, xq):
        """Quantized activation (codes and per-token scales, every member indexed by token on
        axis 0) of this rank's tokens -> the same for all tokens."""
        if isinstance(xq, torch.Tensor):
            return self.all_gather(xq)
        return tuple(self.all_gather(t) for t in xq)


class OverlappedRowParallel:
    """Row-parallel linear + all-reduce with the collective of slab i running on a side stream
    while the GEMM of slab i+1 runs on the compute stream (CUDA only)."""

    def __init__(self, backend, reduce: AllReduce, slabs: int):
        self.backend, self.reduce, self.slabs = backend, reduce, max(1, slabs)
        self.comm_stream = torch.cuda.Stream() if torch.cuda.is_available() and reduce.world > 1 else None

    def __call__(self, x, qw, amax=None) -> torch.Tensor:
        if self.reduce.world == 1:
            return self.backend.linear(x, qw, amax)
        quantized = isinstance(x, tuple)                  # (codes, per-token scales): slice both by token
        rows = x[0].shape[0] if quantized else x.shape[0]
        slabs = min(self.slabs, max(1, rows // 128))
        if slabs == 1 or self.comm_stream is None:
            return self.reduce(self.backend.linear(x, qw, amax))
        bounds = [rows * i // slabs for i in range(slabs + 1)]
        outs = []
        main = torch.cuda.current_stream()
        for i in range(slabs):
            rows_i = slice(bounds[i], bounds[i + 1])
            part = self.backend.linear(tuple(t[rows_i] for t in x) if quantized else x[rows_i], qw, amax)
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ev)
                self.reduce(part)
                part.record_stream(self.comm_stream)
            outs.append(part)
        main.wait_stream(self.comm_stream)
        return torch.cat(outs, dim=0)


# ----------------------------------------------------------------------------- the stack
class DecoderLayer:
    def __init__(self, cfg: StackConfig, weights: dict, backend, world: int = 1, row_parallel=None):
        self.cfg, self.backend, self.world = cfg, backend, world
        self.norm1, self.norm2 = weights["norm1"], weights["norm2"]
        self.wqkv = backend.prepare_weight(weights["wqkv"])
        self.wo = backend.prepare_weight(weights["wo"])
        self.wgu = backend.prepare_weight(weights["wgu"])
        self.wdown = backend.prepare_weight(weights["wdown"])
        self.row_parallel = row_parallel or (lambda x, qw, amax=None: backend.linear(x, qw, amax))
        # Calibrated activation amax per linear input (the `amax` operand of the quantize op is a
        # constant after calibration in the reference flow); filled by a calibration pass.
        self.amax: dict = {}
        self.calibrating = False

    def _amax(self, name: str, x):
        if isinstance(x, tuple):
            return None                                   # already quantized (per-token dynamic scales)
        if self.calibrating and hasattr(self.backend, "measure_amax"):
            m = self.backend.measure_amax(x)
            if m is not None:
                self.amax[name] = m if name not in self.amax else torch.maximum(self.amax[name], m)
        return self.amax.get(name)

    def _norm_amax(self, name: str, h, delta, weight):
        if self.calibrating and hasattr(self.backend, "measure_norm_amax"):
            m = self.backend.measure_norm_amax(h, delta, weight, self.cfg.eps)
            if m is not None:
                self.amax[name] = m if name not in self.amax else torch.maximum(self.amax[name], m)
        return self.amax.get(name)

    def _attention(self, qkv: torch.Tensor) -> torch.Tensor:
        """Attention core on this rank's heads: qkv [T, (q + 2 kv) / W] -> [T, q / W]."""
        cfg, be, w = self.cfg, self.backend, self.world
        if cfg.attention == "fp8_sdpa" and qkv.shape[0] % cfg.seq_len == 0:
            return be.causal_attention(qkv, cfg.n_q // w, cfg.n_kv // w, cfg.head_dim, cfg.seq_len)
        if cfg.attention == "fp8_sdpa" and qkv.shape[0] >= cfg.seq_len:
            raise ValueError(f"{qkv.shape[0]} tokens are not whole sequences of {cfg.seq_len}")
        # fewer tokens than a sequence (a decode step has no key cache here) and the linear-stack form
        col0, heads, rep = (cfg.q_width + cfg.kv_width) // w, cfg.n_q // w, cfg.n_q // cfg.n_kv
        if hasattr(be, "expand_heads_quantize") and not self.calibrating:
            xq = be.expand_heads_quantize(qkv, col0, heads, rep, cfg.head_dim)    # quantized input of the O projection in one pass
            if xq is not None:
                return xq
        return be.expand_heads(qkv, col0, heads, rep, cfg.head_dim)

    def _ffn_act(self, xq):
        """gate/up linear + silu(gate) * up -> input of the down projection (quantized when the
        backend fuses the quantize, else bf16)."""
        be = self.backend
        if hasattr(be, "gate_up_activation") and not self.calibrating:
            act = be.gate_up_activation(xq, self.wgu)     # activation fused into the GEMM epilogue, where the backend has it
            if act is not None:
                return act
        gu = be.matmul(xq, self.wgu)
        act = be.silu_mul_quantize(gu) if hasattr(be, "silu_mul_quantize") and not self.calibrating else None
        return be.silu_mul(gu) if act is None else act

    def forward(self, h: torch.Tensor, delta=None):
        """h: [tokens, hidden] bf16 residual stream; `delta`: output of the previous row-parallel
        linear that has not been added to h yet (the add is fused into the next norm).
        Returns (h, delta) in the same form."""
        cfg, be, w = self.cfg, self.backend, self.world
        h, xq = be.add_norm_quantize(h, delta, self.norm1, cfg.eps, self._norm_amax("qkv", h, delta, self.norm1))
        qkv = be.matmul(xq, self.wqkv)                                   # [T, (q + 2 kv) / W]
        attn = self._attention(qkv)
        delta = self.row_parallel(attn, self.wo, self._amax("o", attn))
        h, xq = be.add_norm_quantize(h, delta, self.norm2, cfg.eps, self._norm_amax("gate_up", h, delta, self.norm2))
        act = self._ffn_act(xq)
        return h, self.row_parallel(act, self.wdown, self._amax("down", act))


    def forward_sharded(self, h: torch.Tensor, delta, comm: ShardedComm):
        """Same layer on a token-sharded residual stream: h, delta are [tokens / W, hidden]; the
        row-parallel partial outputs are computed without their reduction (`partial_linear`) and
        reduce-scattered, the quantized norm outputs are all-gathered."""
        cfg, be, w = self.cfg, self.backend, self.world
        if cfg.mode != "fp8":
            raise ValueError("the token-sharded residual stream is implemented for FP8 stacks")
        h, xq = be.add_norm_quantize(h, delta, self.norm1, cfg.eps)
        qkv = be.matmul(comm.all_gather_quantized(xq), self.wqkv)
        attn = self._attention(qkv)
        delta = comm.reduce_scatter(be.linear(attn, self.wo))
        h, xq = be.add_norm_quantize(h, delta, self.norm2, cfg.eps)
        act = self._ffn_act(comm.all_gather_quantized(xq))
        return h, comm.reduce_scatter(be.linear(act, self.wdown))


    def forward_fused_sharded(self, h: torch.Tensor, xq, rp, next_norm):
        """Token-sharded layer on the fused peer-memory path (tp.FusedRowParallel, sharded): `h` is
        this rank's residual rows (updated in place), `xq` the gathered quantized input of the QKV
        linear.  Each row-parallel GEMM pushes its partial tiles to the owners; one kernel then
        reduces, adds the residual, applies the following RMSNorm, quantizes and gathers.  Returns
        the gathered quantized input of the next layer, or (next_norm None) the full bf16 output."""
        cfg, be, w = self.cfg, self.backend, self.world
        qkv = be.matmul(xq, self.wqkv)
        attn = self._attention(qkv)
        rp.partials_to_owners(attn, self.wo)
        xq = rp.reduce_norm_quantize(h, self.norm2, cfg.eps)
        rp.partials_to_owners(self._ffn_act(xq), self.wdown)
        if next_norm is None:
            return rp.reduce_add(h)
        return rp.reduce_norm_quantize(h, next_norm, cfg.eps)


class DecoderStack:
    """`layers` decoder layers sharing one TP group.  `weights` is an iterable of per-layer dicts
    of full (unsharded) bf16 weights; each is sharded, quantized and dropped."""

    def __init__(self, cfg: StackConfig, weights, backend=None, rank: int = 0, world: int = 1, group=None, slabs: int = 1,
                 fused_rows: int = 0, pull_rows: int = 0, comm=None):
        """`comm`: a tp.CommContext whose CUDA-IPC buffers the fused paths use for their peer memory
        (default: torch's symmetric-memory allocator).  `fused_rows` > 0: row-parallel linears use the fused GEMM + peer-memory all-reduce
        (tp.FusedRowParallel) for up to that many rows; other row counts use NCCL.
        `pull_rows` > 0 (FP8 stacks): forwards of at most that many tokens (decode steps) use the pull
        all-reduce fused with residual add, RMSNorm and quantize (tp.PullRowParallel)."""
        cfg.check(world)
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        self._comm = None
        self._fused = None
        self._pull = None
        self.check_status = True                 # forward() polls the device status word on the fused TP path
        self.backend = backend or CudaBackend(cfg.mode)
        reduce = AllReduce(group) if world > 1 else None
        row_parallel = None
        if world > 1 and fused_rows > 0:
            from .tp import FusedRowParallel

            be = self.backend
            row_parallel = FusedRowParallel(cfg.mode, fused_rows, cfg.hidden, group,
                                            fallback=lambda x, qw, amax=None: reduce(be.linear(x, qw, amax)),
                                            sharded=cfg.mode == "fp8", comm=comm)
            self._fused = row_parallel
        elif world > 1:
            if slabs > 1:
                row_parallel = OverlappedRowParallel(self.backend, reduce, slabs)
            else:
                be = self.backend
                row_parallel = lambda x, qw, amax=None: reduce(be.linear(x, qw, amax))  # noqa: E731
        if world > 1 and pull_rows > 0 and cfg.mode == "fp8":
            from .tp import PullRowParallel

            self._pull = PullRowParallel(cfg.mode, pull_rows, cfg.hidden, group, comm=comm)
        self.layers = [DecoderLayer(cfg, shard_layer_weights(w, cfg, rank, world) if world > 1 else w, self.backend, world,
                                    row_parallel) for w in weights]
        # every weight is quantized and resident from here on: forward() may promise its own GEMM
        # calls that no kernel in flight is still writing them (b200q_cfg::static_weights, per call)
        self._static_weights = isinstance(self.backend, CudaBackend)
        if self._static_weights and torch.cuda.is_available():
            torch.cuda.synchronize()

    def forward(self, h: torch.Tensor, micro_batches: int = 1, sharded=False) -> torch.Tensor:
        """`micro_batches` = 2 (tensor-parallel, CUDA): the tokens are split in two halves that walk
        the layers on two streams, so the collectives of one half run while the other half's
        GEMMs compute.  The result is the same as with one batch: every op is row-wise.
        `sharded`: token-sharded residual stream (reduce-scatter / all-gather of quantized
        activations instead of all-reduce).  True = the fused peer-memory kernels when every
        micro-batch has a multiple of world * 128 tokens, else the all-reduce form; "collectives" =
        the same flow on the process group's reduce-scatter / all-gather (any token count that
        divides by the TP size)."""
        shape = h.shape
        h = h.reshape(-1, shape[-1])
        if sharded not in (False, True, "collectives"):
            raise ValueError(f"sharded must be False, True or 'collectives', got {sharded!r}")
        if self.world == 1:
            sharded = False
        if (self._fused is not None or self._pull is not None) and self.check_status and not (
                h.is_cuda and torch.cuda.is_current_stream_capturing()):
            self.raise_if_device_error()
        if self._pull is not None and h.is_cuda and self._pull.usable(h.shape[0]):
            with capi.gemm_config(static_weights=self._static_weights):
                return self._walk_pull(h).view(shape)
        with capi.gemm_config(static_weights=self._static_weights):
            if micro_batches > 1 and self.world > 1 and h.is_cuda and h.shape[0] >= 2 * 128 * self.world:
                return self._forward_overlapped(h, micro_batches, sharded).view(shape)
            return self._micro_batch(h, sharded).view(shape)

    def raise_if_device_error(self) -> None:
        """The peer-memory reductions skip their work once a bounded device-side wait has run out
        (a peer that never arrived) and the host calls still return success, so their outputs would
        be stale from then on.  This reads the device status word (a synchronising 4-byte copy) and
        raises; `forward` calls it before issuing a step on the fused tensor-parallel path."""
        if capi.device_status(reset=False) != 0:
            raise RuntimeError("a device-side wait for a tensor-parallel peer timed out in an earlier step; "
                               "outputs since then are invalid (b200q_device_status)")

    def _micro_batch(self, h: torch.Tensor, sharded: bool) -> torch.Tensor:
        """All layers over one batch of tokens on the current stream."""
        if sharded is True:
            if self._fused is not None and self._fused.usable(h.shape[0]):
                return self._walk_fused_sharded(h).clone()
            sharded = False
        sharded = bool(sharded)
        return self._finish(*self._walk(self._enter(h, sharded), None, sharded), sharded)

    def _walk_pull(self, h: torch.Tensor) -> torch.Tensor:
        """A few tokens (decode): replicated residual stream, every row-parallel linear ends in the
        pull all-reduce fused with the next norm + quantize."""
        be, cfg = self.backend, self.cfg
        h = h.clone()                                     # updated in place from here on
        _, xq = be.add_norm_quantize(h, None, self.layers[0].norm1, cfg.eps)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].norm1 if i + 1 < len(self.layers) else None
            xq = layer.forward_fused_sharded(h, xq, self._pull, nxt)
        return xq

    def _walk_fused_sharded(self, h: torch.Tensor) -> torch.Tensor:
        comm, be, cfg = self._comm_obj(), self.backend, self.cfg
        h = comm.shard(h).clone()                         # updated in place from here on
        _, xq = be.add_norm_quantize(h, None, self.layers[0].norm1, cfg.eps)
        xq = comm.all_gather_quantized(xq)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].norm1 if i + 1 < len(self.layers) else None
            xq = layer.forward_fused_sharded(h, xq, self._fused, nxt)
        return xq

    # one micro-batch: enter (take this rank's tokens), walk the layers, finish (last residual add
    # and, token-sharded, the all-gather of the bf16 result)
    def _comm_obj(self) -> ShardedComm:
        if self._comm is None:
            self._comm = ShardedComm(self.group)
        return self._comm

    def _enter(self, h: torch.Tensor, sharded: bool) -> torch.Tensor:
        if not sharded:
            return h
        if h.shape[0] % self.world:
            raise ValueError(f"{h.shape[0]} tokens do not divide over {self.world} ranks")
        return self._comm_obj().shard(h)

    def _walk(self, h, delta, sharded: bool):
        for layer in self.layers:
            h, delta = layer.forward_sharded(h, delta, self._comm_obj()) if sharded else layer.forward(h, delta)
        return h, delta

    def _finish(self, h, delta, sharded: bool) -> torch.Tensor:
        out = self.backend.add(h, delta)
        return self._comm_obj().all_gather(out) if sharded else out

    def _forward_overlapped(self, h: torch.Tensor, n: int, sharded: bool = False) -> torch.Tensor:
        main = torch.cuda.current_stream()
        if getattr(self, "_streams", None) is None or len(self._streams) != n:
            self._streams = [torch.cuda.Stream() for _ in range(n)]
        rows = h.shape[0]
        step = (rows // n + 127) // 128 * 128
        chunks = [h[i * step:min(rows, (i + 1) * step)] for i in range(n)]
        for st in self._streams:
            st.wait_stream(main)
        fused = sharded is True and self._fused is not None and all(self._fused.usable(c.shape[0]) for c in chunks)
        sharded = sharded == "collectives"
        if fused:
            parts = self._overlapped_fused_sharded(chunks)
        else:
            parts = [self._enter(c, sharded) for c in chunks]
            deltas = [None] * n
            comm = self._comm_obj() if sharded else None
            for layer in self.layers:
                for i, st in enumerate(self._streams):
                    with torch.cuda.stream(st):
                        if sharded:
                            parts[i], deltas[i] = layer.forward_sharded(parts[i], deltas[i], comm)
                        else:
                            parts[i], deltas[i] = layer.forward(parts[i], deltas[i])
            for i, st in enumerate(self._streams):
                with torch.cuda.stream(st):
                    parts[i] = self._finish(parts[i], deltas[i], sharded)
        for i, st in enumerate(self._streams):
            parts[i].record_stream(main)
            main.wait_stream(st)
        h.record_stream(self._streams[0])
        return torch.cat(parts, dim=0)

    def _overlapped_fused_sharded(self, chunks):
        comm, be, cfg = self._comm_obj(), self.backend, self.cfg
        hs, xqs = [None] * len(chunks), [None] * len(chunks)
        for i, st in enumerate(self._streams):
            with torch.cuda.stream(st):
                hs[i] = comm.shard(chunks[i]).clone()
                _, xq = be.add_norm_quantize(hs[i], None, self.layers[0].norm1, cfg.eps)
                xqs[i] = comm.all_gather_quantized(xq)
        for li, layer in enumerate(self.layers):
            nxt = self.layers[li + 1].norm1 if li + 1 < len(self.layers) else None
            for i, st in enumerate(self._streams):
                with torch.cuda.stream(st):
                    xqs[i] = layer.forward_fused_sharded(hs[i], xqs[i], self._fused, nxt)
        return xqs

    __call__ = forward

    def calibrate(self, h: torch.Tensor) -> torch.Tensor:
        """One forward that records the activation amax in front of every linear; later forwards
        use the recorded values as static quantizer inputs (NVFP4 only; FP8 is per-token dynamic)."""
        for layer in self.layers:
            layer.calibrating = True
        try:
            return self.forward(h)
        finally:
            for layer in self.layers:
                layer.calibrating = False


def random_layer_weights(cfg: StackConfig, seed: int, device="cuda", dtype=torch.bfloat16):
    """Generator of per-layer full weights ~ N(0, 0.02), RMSNorm weights = 1 (same values on
    every rank for the same seed)."""
    g = torch.Generator(device=device).manual_seed(seed)
    for _ in range(cfg.layers):
        def rnd(r, c):
            return (torch.randn(r, c, device=device, dtype=torch.float32, generator=g) * 0.02).to(dtype)
        yield {
            "norm1": torch.ones(cfg.hidden, device=device, dtype=dtype), "norm2": torch.ones(cfg.hidden, device=device, dtype=dtype),
            "wqkv": rnd(cfg.q_width + 2 * cfg.kv_width, cfg.hidden), "wo": rnd(cfg.hidden, cfg.q_width),
            "wgu": rnd(2 * cfg.ffn, cfg.hidden), "wdown": rnd(cfg.hidden, cfg.ffn),
        }
