"""Tensor-parallel host logic on CPU: two gloo ranks (spawned processes, FileStore rendezvous on
127.0.0.1-free file paths) run the stack's layer logic with a backend made of the CPU oracle, the
`tensorrt::fused_nccl_all_reduce` op is checked against its known answer, and host-side failure
detection (shape mismatch across ranks, a rank that never joins) is exercised without any GPU."""
import os
import sys
import tempfile
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBackend:
    """CPU stand-in for the device kernels, built from the oracle (tests only)."""

    def __init__(self, mode):
        import oracle as o

        self.o, self.mode = o, mode

    def prepare_weight(self, w):
        return w

    def linear(self, x, w, amax=None):
        o = self.o
        y = o.fp8_linear_ref(x, w) if self.mode == "fp8" else o.nvfp4_linear_ref(x, w)
        return y.to(x.dtype)

    def matmul(self, xq, w):
        return self.linear(xq, w)

    def add_norm_quantize(self, h, delta, w, eps, amax=None):
        h_new = h if delta is None else h + delta
        return h_new, self.o.rms_norm_ref(h_new, w, eps)

    def rms_norm(self, x, w, eps):
        return self.o.rms_norm_ref(x, w, eps)

    def causal_attention(self, qkv, n_q, n_kv, head_dim, seq_len):
        return self.o.causal_attention_ref(qkv, n_q, n_kv, head_dim, seq_len)

    def silu_mul(self, gu):
        f = gu.shape[-1] // 2
        return (torch.nn.functional.silu(gu[..., :f].float()) * gu[..., f:].float()).to(gu.dtype)

    def add(self, a, b):
        return a + b

    def expand_heads(self, src, col0, heads_out, rep, head_dim):
        v = src[..., col0:col0 + (heads_out // rep) * head_dim]
        return v.reshape(*v.shape[:-1], heads_out // rep, 1, head_dim).expand(
            *v.shape[:-1], heads_out // rep, rep, head_dim).reshape(*v.shape[:-1], -1).contiguous()


def _layer_weights(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(cfg.layers):
        rnd = lambda r, c: (torch.randn(r, c, generator=g) * 0.02).bfloat16()  # noqa: E731
        out.append({"norm1": torch.ones(cfg.hidden).bfloat16(), "norm2": torch.ones(cfg.hidden).bfloat16(),
                    "wqkv": rnd(cfg.q_width + 2 * cfg.kv_width, cfg.hidden), "wo": rnd(cfg.hidden, cfg.q_width),
                    "wgu": rnd(2 * cfg.ffn, cfg.hidden), "wdown": rnd(cfg.hidden, cfg.ffn)})
    return out


def _init(rank, world, store_path, timeout_s=60):
    sys.path.insert(0, ROOT)
    store = dist.FileStore(store_path, world)
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=timedelta(seconds=timeout_s))


def _worker_stack(rank, world, store_path, mode, out_path):
    _init(rank, world, store_path)
    import oracle as o
    import tensorrt_b200  # registers tensorrt::fused_nccl_all_reduce
    from tensorrt_b200.stack import DecoderStack, StackConfig
    from tensorrt_b200.tp import group_name_of

    # 1. the op, known answer: sum(fill(rank + 1)) == W (W + 1) / 2
    t = torch.full((1, 4), float(rank + 1))
    r = torch.ops.tensorrt.fused_nccl_all_reduce(t, "sum", group_name_of())
    assert torch.allclose(r, torch.full((1, 4), world * (world + 1) / 2), atol=1e-3, rtol=1e-3)
    assert torch.equal(t, torch.full((1, 4), float(rank + 1))), "the op must not modify its input"
    r = torch.ops.tensorrt.fused_nccl_all_reduce(t, "max", group_name_of())
    assert torch.equal(r, torch.full((1, 4), float(world)))

    # 1b. group resolution without a pinned name: exactly one gloo group is registered here
    from tensorrt_b200.tp import auto_group_name, probe_group_names, resolve_group

    names = probe_group_names("gloo")
    assert names == [group_name_of()] and auto_group_name("gloo") == names[0]
    assert probe_group_names("nccl") == []
    assert resolve_group(names[0]) is not None
    sub = dist.new_group(list(range(world)))                 # a second group: no automatic choice any more
    try:
        auto_group_name("gloo")
    except RuntimeError as e:
        assert "pass the group name" in str(e)
    else:
        raise AssertionError("two registered groups must not be resolved automatically")
    r = torch.ops.tensorrt.fused_nccl_all_reduce(t, "sum", group_name_of(sub))
    assert torch.allclose(r, torch.full((1, 4), world * (world + 1) / 2))

    # 2. the TP stack against the oracle's TP restatement (same arithmetic -> identical) and
    #    against the unsharded layer (different summation order / activation slices -> close)
    cfg = StackConfig(hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, layers=2, mode=mode)
    weights = _layer_weights(cfg, seed=4)
    g = torch.Generator().manual_seed(40)
    h = torch.randn(2, 8, cfg.hidden, generator=g).bfloat16()
    stack = DecoderStack(cfg, weights, backend=OracleBackend(mode), rank=rank, world=world)
    y = stack(h)
    ref_tp, ref_1 = h, h
    for w in weights:
        ref_tp = o.decoder_layer_ref(ref_tp, w, cfg.n_q, cfg.n_kv, cfg.head_dim, mode, world=world)
        ref_1 = o.decoder_layer_ref(ref_1, w, cfg.n_q, cfg.n_kv, cfg.head_dim, mode, world=1)
    assert torch.equal(y, ref_tp), o.rel_l2(y.float(), ref_tp.float())
    assert o.rel_l2(y.float(), ref_1.float()) < (3e-2 if mode == "fp8" else 1e-1)
    if mode == "fp8":
        # token-sharded residual stream: reduce-scatter + all-gather of the norm outputs; every
        # token sees the same arithmetic as with the all-reduce
        y_sharded = stack.forward(h, sharded="collectives")
        assert torch.equal(y_sharded, ref_tp), o.rel_l2(y_sharded.float(), ref_tp.float())
        try:
            stack.forward(h[:, :7], sharded="collectives")       # 14 tokens over 2 ranks is fine, 2 x 7 ...
            stack.forward(h[:1, :7], sharded="collectives")      # ... 7 tokens are not
        except ValueError as e:
            assert "do not divide" in str(e)
        else:
            raise AssertionError("ragged token count not rejected")
        # sharded=True asks for the fused peer-memory kernels; without them (CPU) it is the all-reduce form
        assert torch.equal(stack.forward(h, sharded=True), ref_tp)
        # causal FP8 attention as the attention core (2 sequences of 8 tokens), every rank on its own heads
        from dataclasses import replace

        cfg_a = replace(cfg, attention="fp8_sdpa", seq_len=8)
        stack_a = DecoderStack(cfg_a, weights, backend=OracleBackend(mode), rank=rank, world=world)
        ref_a = h.reshape(-1, cfg.hidden)
        for w in weights:
            ref_a = o.decoder_layer_ref(ref_a, w, cfg.n_q, cfg.n_kv, cfg.head_dim, mode, world=world, attention="fp8_sdpa", seq_len=8)
        for form in (False, "collectives"):
            assert torch.equal(stack_a.forward(h, sharded=form).reshape(-1, cfg.hidden), ref_a)
        assert not torch.equal(ref_a, ref_tp.reshape(-1, cfg.hidden))
        try:
            DecoderStack(replace(cfg, attention="fp8_sdpa", seq_len=5), weights, backend=OracleBackend(mode), rank=rank,
                         world=world).forward(h)
        except ValueError as e:
            assert "whole sequences" in str(e)
        else:
            raise AssertionError("16 tokens are not whole sequences of 5")
    if rank == 0:
        torch.save(y, out_path)
    dist.barrier()
    dist.destroy_process_group()


def _worker_mismatch(rank, world, store_path):
    _init(rank, world, store_path)
    from tensorrt_b200.tp import ShapeMismatchError, check_same_shape

    check_same_shape(torch.zeros(4, 8))                      # same everywhere: passes
    bad = torch.zeros(4, 8 if rank == 0 else 16)
    try:
        check_same_shape(bad)
    except ShapeMismatchError as e:
        assert "differ across ranks" in str(e)
    else:
        raise AssertionError("mismatch not detected")
    dist.barrier()
    dist.destroy_process_group()


def _worker_eight_ranks(rank, world, store_path):
    _init(rank, world, store_path, timeout_s=120)
    import oracle as o
    from tensorrt_b200.stack import DecoderStack, StackConfig

    cfg = StackConfig(hidden=256, n_q=8, n_kv=8, head_dim=32, ffn=512, layers=2, mode="fp8")
    weights = _layer_weights(cfg, seed=4)
    g = torch.Generator().manual_seed(41)
    h = torch.randn(2, 16, cfg.hidden, generator=g).bfloat16()
    stack = DecoderStack(cfg, weights, backend=OracleBackend("fp8"), rank=rank, world=world)
    y = stack(h)
    # the process-group form of the token-sharded flow: the same sums on the same backend, so the same bits
    assert torch.equal(stack.forward(h, sharded="collectives"), y)
    ref = h
    for w in weights:
        ref = o.decoder_layer_ref(ref, w, cfg.n_q, cfg.n_kv, cfg.head_dim, "fp8", world=world)
    # the oracle sums the 8 partials in fp32 and rounds once; a bf16 collective rounds at every hop,
    # and the FP8 re-quantization after each reduction amplifies that: close, not equal
    assert o.rel_l2(y.float(), ref.float()) < 5e-2
    dist.barrier()
    dist.destroy_process_group()


def _worker_missing_peer(rank, world, store_path):
    # rank 1 never joins: rank 0's rendezvous must end with an error within its timeout
    if rank == 1:
        return
    try:
        _init(rank, world, store_path, timeout_s=3)
        dist.barrier()
    except Exception as e:  # DistStoreError / RuntimeError depending on where it times out
        assert "imeout" in str(e) or "timed out" in str(e).lower() or "store" in str(e).lower(), str(e)
    else:
        raise AssertionError("rendezvous with a missing peer did not fail")


def _worker_row_parallel_bias(rank, world, store_path):
    """A checkpoint-loaded row-parallel linear keeps its bias on rank 0 only ("linear, then all-reduce"
    adds it once); the fused path adds the bias after the sum on the owner of each row and needs the
    full bias everywhere.  Both routes must give the same result."""
    _init(rank, world, store_path)
    import oracle as o
    from tensorrt_b200.tp import replicate_row_parallel_bias

    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(8, 64, generator=g).bfloat16(), (torch.randn(16, 64, generator=g) * 0.1).bfloat16()
    full_bias = torch.randn(16, generator=g).bfloat16()
    ks = 64 // world
    xs, wr = x[:, rank * ks:(rank + 1) * ks].contiguous(), w[:, rank * ks:(rank + 1) * ks].contiguous()
    loaded = full_bias.clone() if rank == 0 else None                     # what checkpoint.load_quantized_linears returns
    # route 1: linear (+ the bias where it lives), then all-reduce
    part = o.fp8_linear_ref(xs, wr, loaded)
    total = part.clone()
    dist.all_reduce(total)
    # route 2 (fused convention): replicate the bias, sum the bias-free partials, add the bias once
    rep = replicate_row_parallel_bias(loaded)
    assert rep is not None and torch.equal(rep, full_bias)
    bare = o.fp8_linear_ref(xs, wr)
    dist.all_reduce(bare)
    assert torch.allclose(bare + rep.float(), total, atol=1e-5)
    # already replicated: returned as is; absent everywhere: None; a bias on a rank other than 0 only: error
    assert replicate_row_parallel_bias(full_bias) is full_bias
    assert replicate_row_parallel_bias(None) is None
    try:
        replicate_row_parallel_bias(full_bias if rank == 1 else None)
    except ValueError as e:
        assert "rank 0" in str(e)
    else:
        raise AssertionError("a bias that lives on rank 1 only was accepted")
    dist.barrier()
    dist.destroy_process_group()


def _spawn(fn, world, *args):
    with tempfile.TemporaryDirectory() as d:
        store = os.path.join(d, "store")
        mp.spawn(fn, args=(world, store, *args), nprocs=world, join=True)


@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
def test_two_rank_stack_and_all_reduce_op(mode, tmp_path):
    out = str(tmp_path / "y.pt")
    _spawn(_worker_stack, 2, mode, out)
    assert torch.load(out).shape == (2, 8, 256)


def test_eight_rank_collectives_form_equals_all_reduce_form():
    _spawn(_worker_eight_ranks, 8)


def test_shape_mismatch_is_detected_on_the_host():
    _spawn(_worker_mismatch, 2)


def test_row_parallel_bias_conventions_agree():
    _spawn(_worker_row_parallel_bias, 2)


def test_missing_peer_times_out_on_the_host():
    _spawn(_worker_missing_peer, 2)


def test_single_process_all_reduce_is_identity(b200):
    t = torch.arange(8.0)
    r = torch.ops.tensorrt.fused_nccl_all_reduce(t, "sum", "default")
    assert torch.equal(r, t) and r.data_ptr() != t.data_ptr()
    with pytest.raises(ValueError):
        torch.ops.tensorrt.fused_nccl_all_reduce(t, "xor", "default")


def test_sharding_helpers():
    from tensorrt_b200.stack import StackConfig, shard_layer_weights
    from tensorrt_b200.tp import shard_cols, shard_rows

    w = torch.arange(8 * 6.0).view(8, 6)
    assert torch.equal(torch.cat([shard_rows(w, r, 4) for r in range(4)]), w)
    assert torch.equal(torch.cat([shard_cols(w, r, 3) for r in range(3)], dim=1), w)
    with pytest.raises(ValueError):
        shard_rows(w, 0, 3)
    cfg = StackConfig(hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, layers=1)
    lw = _layer_weights(cfg, 1)[0]
    parts = [shard_layer_weights(lw, cfg, r, 2) for r in range(2)]
    assert parts[0]["wqkv"].shape == (256, 256) and parts[0]["wo"].shape == (256, 128)
    assert parts[0]["wgu"].shape == (512, 256) and parts[0]["wdown"].shape == (256, 256)
    assert torch.equal(torch.cat([p["wo"] for p in parts], dim=1), lw["wo"])
    with pytest.raises(ValueError):
        cfg.check(world=4)          # 2 kv heads do not split over 4 ranks
