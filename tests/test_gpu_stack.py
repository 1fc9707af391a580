"""GPU parity of the decoder linear stack (glue kernels + quantized linears) against the oracle,
on one GPU and, when two are visible, on two NCCL ranks."""
import os
import sys
import tempfile

import pytest
import torch

import oracle as o

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _weights(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(cfg.layers):
        rnd = lambda r, c: (torch.randn(r, c, generator=g) * 0.02).bfloat16()  # noqa: E731
        out.append({"norm1": (1 + 0.1 * torch.randn(cfg.hidden, generator=g)).bfloat16(),
                    "norm2": (1 + 0.1 * torch.randn(cfg.hidden, generator=g)).bfloat16(),
                    "wqkv": rnd(cfg.q_width + 2 * cfg.kv_width, cfg.hidden), "wo": rnd(cfg.hidden, cfg.q_width),
                    "wgu": rnd(2 * cfg.ffn, cfg.hidden), "wdown": rnd(cfg.hidden, cfg.ffn)})
    return out


def _to(ws, dev):
    return [{k: v.to(dev) for k, v in w.items()} for w in ws]


def test_glue_kernels(b200):
    capi = b200.capi
    g = torch.Generator().manual_seed(1)
    x = torch.randn(37, 1024, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(1024, generator=g)).bfloat16()
    y = capi.rms_norm(x.cuda(), w.cuda(), 1e-5)
    assert o.rel_l2(y.float().cpu(), o.rms_norm_ref(x, w).float()) < 4e-3
    for cols in (8, 4096, 8200):                               # register-resident and streamed variants
        xx = torch.randn(5, cols, generator=g).bfloat16()
        ww = torch.ones(cols).bfloat16()
        assert o.rel_l2(capi.rms_norm(xx.cuda(), ww.cuda()).float().cpu(), o.rms_norm_ref(xx, ww).float()) < 4e-3
    gu = torch.randn(33, 2 * 520, generator=g).bfloat16()
    ref = (torch.nn.functional.silu(gu[:, :520].float()) * gu[:, 520:].float()).bfloat16()
    assert o.rel_l2(capi.silu_mul(gu.cuda()).float().cpu(), ref.float()) < 4e-3
    a, b = torch.randn(64, 72, generator=g).bfloat16(), torch.randn(64, 72, generator=g).bfloat16()
    assert torch.equal(capi.add(a.cuda(), b.cuda()).cpu(), (a.float() + b.float()).bfloat16())
    src = torch.randn(9, 6 * 64, generator=g).bfloat16()          # [q: 4 heads | k: 1 | v: 1] of dim 64
    out = capi.expand_heads(src.cuda(), 5 * 64, 4, 4, 64).cpu()
    assert torch.equal(out, src[:, 5 * 64:].repeat(1, 4))
    src = torch.randn(9, 8 * 64, generator=g).bfloat16()          # 2 kv heads, each repeated twice
    out = capi.expand_heads(src.cuda(), 6 * 64, 4, 2, 64).cpu()
    v = src[:, 6 * 64:].view(9, 2, 1, 64).expand(9, 2, 2, 64).reshape(9, 256)
    assert torch.equal(out, v)


@pytest.mark.parametrize("rows,kv_heads,rep,hd,q_cols", [(9, 2, 2, 64, 384), (300, 8, 8, 128, 8192), (1000, 1, 8, 128, 1024),
                                                         (33, 4, 1, 32, 0), (5, 16, 2, 128, 256)])
def test_expand_heads_with_fused_quantize_is_bit_identical(b200, rows, kv_heads, rep, hd, q_cols):
    """The repeated-head expansion and the per-token FP8 quantize in front of the O projection in one kernel:
    codes and scales equal those of the two separate kernels (an all-zero token included)."""
    capi = b200.capi
    g = torch.Generator().manual_seed(rows + hd)
    width = q_cols + 2 * kv_heads * hd                  # [q | k | v] columns of a QKV output
    src = (torch.randn(rows, width, generator=g) * 2).bfloat16()
    src[rows // 2] = 0
    col0 = q_cols + kv_heads * hd
    codes, scales = capi.expand_heads_fp8_quantize(src.cuda(), col0, kv_heads * rep, rep, hd)
    c_ref, s_ref = capi.fp8_quantize(capi.expand_heads(src.cuda(), col0, kv_heads * rep, rep, hd), None)
    assert codes.shape == (rows, kv_heads * rep * hd) and torch.equal(codes, c_ref) and torch.equal(scales, s_ref)
    with pytest.raises(b200.B200QError):
        capi.expand_heads_fp8_quantize(torch.zeros(2, 4096, dtype=torch.bfloat16, device="cuda"), 0, 32, 1, 128)   # kv slice beyond 2048


# from 8 rows per SM and 4096 columns on: persistent CTAs fed by a ring of 4096-column chunks (1, 2 with a ragged
# second, 4 ragged, 7 and 8 chunks per row; CTAs that walk 4 and 5 rows)
@pytest.mark.parametrize("rows,f", [(1, 16), (33, 528), (64, 3584), (17, 14336), (5, 28672), (3, 32768),
                                    (1184, 4096), (1400, 4112), (1190, 14336), (1200, 28672), (1185, 32768)])
def test_fused_silu_mul_quantize_is_bit_identical(b200, rows, f):
    """silu(gate) * up + per-token FP8 quantize in one kernel: codes and scales equal those of the
    two separate kernels bit for bit (same bf16 rounding point, same division), and dequantize to
    the oracle's activation."""
    capi = b200.capi
    g = torch.Generator().manual_seed(rows + f)
    gu = (torch.randn(rows, 2 * f, generator=g) * 2).bfloat16()
    if f > 8:
        gu[0] = 0                                     # an all-zero token: scale 1, codes 0
    codes, scales = capi.silu_mul_fp8_quantize(gu.cuda())
    c_ref, s_ref = capi.fp8_quantize(capi.silu_mul(gu.cuda()), None)
    assert codes.shape == (rows, f) and scales.shape == (rows,)
    assert torch.equal(scales, s_ref) and torch.equal(codes, c_ref)
    ref = torch.nn.functional.silu(gu[:, :f].float()) * gu[:, f:].float()
    assert o.rel_l2(capi.fp8_dequantize(codes, scales, torch.float32).cpu(), ref) < 4e-2
    with pytest.raises(b200.B200QError):
        capi.silu_mul_fp8_quantize(torch.zeros(2, 2 * 32776, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("cols", [64, 4096, 8192, 12288])
def test_fused_add_norm_quantize(b200, cols):
    """h + delta, RMSNorm and per-token FP8 quantize in one kernel against the three separate
    kernels (same rounding points: identical h, codes equal wherever the norm's fp32 sum order
    does not flip a bf16 rounding) and against the oracle."""
    capi = b200.capi
    g = torch.Generator().manual_seed(cols)
    h = torch.randn(37, cols, generator=g).bfloat16()
    d = (torch.randn(37, cols, generator=g) * 0.3).bfloat16()
    w = (1 + 0.1 * torch.randn(cols, generator=g)).bfloat16()
    h_new, codes, scales = capi.add_rms_norm_fp8_quantize(h.cuda(), d.cuda(), w.cuda(), 1e-5)
    h_ref = capi.add(h.cuda(), d.cuda())
    assert torch.equal(h_new, h_ref)
    c_ref, s_ref = capi.fp8_quantize(capi.rms_norm(h_ref, w.cuda(), 1e-5), None)
    assert torch.allclose(scales, s_ref, rtol=1e-2)
    assert (codes != c_ref).float().mean().item() < 2e-2
    x_oracle = o.rms_norm_ref(h + d, w)
    deq = capi.fp8_dequantize(codes, scales, torch.float32).cpu()
    assert o.rel_l2(deq, x_oracle.float()) < 4e-2
    # without a delta: h passes through untouched
    h2, codes2, scales2 = capi.add_rms_norm_fp8_quantize(h.cuda(), None, w.cuda(), 1e-5)
    assert h2.data_ptr() == h2.data_ptr() and torch.equal(h2.cpu(), h)
    c3, s3 = capi.fp8_quantize(capi.rms_norm(h.cuda(), w.cuda(), 1e-5), None)
    assert (codes2 != c3).float().mean().item() < 2e-2


@pytest.mark.parametrize("cols", [64, 1040, 4096, 8192, 12288])
@pytest.mark.parametrize("rows", [1184, 2501])
def test_fused_add_norm_quantize_many_tokens(b200, rows, cols):
    """From 8 rows per SM on, the kernel is the persistent one fed through a shared-memory ring of rows
    (where a row fits the ring): bit-identical with the one-CTA-per-row form run on slices of the same
    input, with and without delta, repeatedly (the ring's barriers start from scratch every launch)."""
    capi = b200.capi
    g = torch.Generator().manual_seed(rows + cols)
    h = torch.randn(rows, cols, generator=g).bfloat16().cuda()
    d = (torch.randn(rows, cols, generator=g) * 0.3).bfloat16().cuda()
    w = (1 + 0.1 * torch.randn(cols, generator=g)).bfloat16().cuda()
    # slices of 300 to 900 rows: one CTA per row there (fewer rows would split a row over a cluster,
    # which sums the squares in another order)
    edges = list(range(0, rows - 300, 400)) + [rows]
    for delta in (d, None):
        parts = [capi.add_rms_norm_fp8_quantize(h[a:b].clone(), None if delta is None else delta[a:b], w, 1e-5)
                 for a, b in zip(edges[:-1], edges[1:])]
        for _ in range(2):
            h_new, codes, scales = capi.add_rms_norm_fp8_quantize(h.clone(), delta, w, 1e-5)
            assert torch.equal(h_new, torch.cat([p[0] for p in parts]))
            assert torch.equal(codes, torch.cat([p[1] for p in parts]))
            assert torch.equal(scales, torch.cat([p[2] for p in parts]))
    assert capi.device_status() == 0


@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
def test_stack_matches_oracle_single_gpu(b200, mode):
    from tensorrt_b200.stack import DecoderStack, StackConfig

    cfg = StackConfig(hidden=512, n_q=8, n_kv=2, head_dim=64, ffn=1024, layers=2, mode=mode)
    ws = _weights(cfg, 7)
    g = torch.Generator().manual_seed(70)
    h = torch.randn(3, 50, cfg.hidden, generator=g).bfloat16()
    y = DecoderStack(cfg, _to(ws, "cuda"))(h.cuda())
    torch.cuda.synchronize()
    assert b200.capi.device_status() == 0
    ref = h
    for w in ws:
        ref = o.decoder_layer_ref(ref, w, cfg.n_q, cfg.n_kv, cfg.head_dim, mode)
    assert y.shape == h.shape
    # bf16 intermediates round differently on the two sides; the quantized linears then see
    # slightly different inputs, so the tolerance is looser than for a single GEMM
    assert o.rel_l2(y.float().cpu(), ref.float()) < (2e-2 if mode == "fp8" else 6e-2)


def test_stack_with_fp8_attention_matches_oracle(b200):
    """Attention core = causal FP8 SDPA (b200q_fp8_sdpa on Q, K, V quantized per tensor) instead of the
    identity stand-in: 3 sequences of 128 tokens through 2 layers against the oracle's layer with the
    same attention core; a 5-token forward (a decode step: no key cache here) takes the stand-in."""
    from tensorrt_b200.stack import DecoderStack, StackConfig

    cfg = StackConfig(hidden=512, n_q=8, n_kv=2, head_dim=64, ffn=1024, layers=2, mode="fp8", attention="fp8_sdpa", seq_len=128)
    ws = _weights(cfg, 9)
    g = torch.Generator().manual_seed(71)
    h = torch.randn(3 * 128, cfg.hidden, generator=g).bfloat16()
    stack = DecoderStack(cfg, _to(ws, "cuda"))
    y = stack(h.cuda())
    torch.cuda.synchronize()
    assert b200.capi.device_status() == 0
    ref, ref_id = h, h
    for w in ws:
        ref = o.decoder_layer_ref(ref, w, cfg.n_q, cfg.n_kv, cfg.head_dim, "fp8", attention="fp8_sdpa", seq_len=128)
        ref_id = o.decoder_layer_ref(ref_id, w, cfg.n_q, cfg.n_kv, cfg.head_dim, "fp8")
    err = o.rel_l2(y.float().cpu(), ref.float())
    assert err < 2e-2, err
    assert o.rel_l2(ref_id.float(), ref.float()) > 10 * err          # the two attention cores are far apart
    assert stack(h[:5].cuda()).shape == (5, cfg.hidden)
    with pytest.raises(ValueError):
        stack(h[:200].cuda())                                        # 200 tokens are not whole sequences of 128


def _tp_worker(rank, world, store_path, out_path, slabs, fused, micro, sharded):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from tensorrt_b200.stack import DecoderStack, StackConfig

    torch.cuda.set_device(rank)
    store = dist.FileStore(store_path, world)
    dist.init_process_group("nccl", store=store, rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dist.barrier()
    cfg = StackConfig(hidden=512, n_q=8, n_kv=2, head_dim=64, ffn=1024, layers=2, mode="fp8")
    ws = _weights(cfg, 7)
    g = torch.Generator().manual_seed(70)
    h = torch.randn(4, 128, cfg.hidden, generator=g).bfloat16()
    # known answer of the op itself on NCCL
    t = torch.full((1, 4), float(rank + 1), device="cuda")
    import tensorrt_b200
    from tensorrt_b200.tp import group_name_of

    r = torch.ops.tensorrt.fused_nccl_all_reduce(t, "sum", group_name_of())
    assert torch.allclose(r.cpu(), torch.full((1, 4), world * (world + 1) / 2), atol=1e-3, rtol=1e-3)
    comm = None
    if fused == "comm":
        # peer buffers from the library's own CUDA-IPC context instead of torch's symmetric memory
        from tensorrt_b200.tp import CommContext

        comm = CommContext()
    stack = DecoderStack(cfg, _to(ws, "cuda"), rank=rank, world=world, slabs=slabs, fused_rows=512 if fused else 0,
                         pull_rows=64 if fused else 0, comm=comm)
    if sharded and not fused:
        sharded = "collectives"                  # the process group's reduce-scatter / all-gather
    y = stack.forward(h.cuda(), micro, sharded)
    y2 = stack.forward(h.cuda(), micro, sharded)  # a second pass reuses the peer buffers and flag epochs
    assert torch.equal(y, y2)
    if sharded:
        # same arithmetic per token as the all-reduce form; only the order of the cross-rank sum
        # may differ (NCCL reduce-scatter vs all-reduce), so compare closely, not bitwise
        y_ar = stack.forward(h.cuda(), micro, False)
        err = (y.float() - y_ar.float()).norm() / y_ar.float().norm()
        assert err < 2e-3, float(err)
    if fused:
        # a decode-sized forward takes the pull all-reduce; eagerly and as a replayed CUDA graph (no
        # collective-library call inside the step), against the all-reduce form of the same stack
        hd = h.cuda()[0, :48].contiguous()
        yd = stack.forward(hd)
        stack._pull, keep = None, stack._pull
        yd_ref = stack.forward(hd)
        stack._pull = keep
        err = (yd.float() - yd_ref.float()).norm() / yd_ref.float().norm()
        assert err < 2e-3, float(err)
        torch.cuda.synchronize()
        dist.barrier()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                yg = stack.forward(hd)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(yg, yd)
    torch.cuda.synchronize()
    assert tensorrt_b200.capi.device_status() == 0
    if rank == 0:
        torch.save(y.cpu(), out_path)
    dist.barrier()
    if comm is not None:
        del stack
        comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("slabs,fused,micro,sharded", [
    (1, False, 1, False), (2, False, 1, False), (1, True, 1, False), (1, False, 2, False), (1, True, 2, False),
    (1, False, 1, True), (1, True, 1, True), (1, False, 2, True), (1, True, 2, True), (1, "comm", 2, True)])
def test_tp2_stack_matches_oracle(b200, slabs, fused, micro, sharded):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from tensorrt_b200.stack import StackConfig

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "y.pt")
        mp.spawn(_tp_worker, args=(2, os.path.join(d, "store"), out, slabs, fused, micro, sharded), nprocs=2, join=True)
        y = torch.load(out)
    cfg = StackConfig(hidden=512, n_q=8, n_kv=2, head_dim=64, ffn=1024, layers=2, mode="fp8")
    ws = _weights(cfg, 7)
    g = torch.Generator().manual_seed(70)
    h = torch.randn(4, 128, cfg.hidden, generator=g).bfloat16()
    ref = h
    for w in ws:
        ref = o.decoder_layer_ref(ref, w, cfg.n_q, cfg.n_kv, cfg.head_dim, "fp8", world=2)
    assert o.rel_l2(y.float(), ref.float()) < 2e-2
