"""GPU parity of the tcgen05 GEMMs and the fused linear layers against the oracle's fp32
dequantize-then-matmul reference.  Tolerance: rel-L2 <= 1e-2 (the output is rounded to bf16)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as o

pytestmark = pytest.mark.gpu
G = Path(__file__).parent / "golden"
TOL = 1e-2


@pytest.fixture(scope="module")
def capi(b200):
    return b200.capi


@pytest.fixture(autouse=True)
def _status(capi):
    yield
    assert capi.device_status() == 0, "a GEMM reported a device-side wait that gave up"


def _inputs(M, N, K, seed, bias=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    b = (torch.randn(N, generator=g) * 0.01).bfloat16() if bias else None
    return x, w, b


def _ref_fp8(x, w, b):
    xc, xs = o.fp8_quantize(x, o.row_amax(x))
    wc, ws = o.fp8_quantize(w, o.row_amax(w))
    # fp32 matmul on the device (TF32 off) of the exactly dequantized operands
    xd, wd = o.fp8_dequantize(xc, xs).cuda(), o.fp8_dequantize(wc, ws).cuda()
    y = xd @ wd.t()
    if b is not None:
        y = y + b.float().cuda()
    return (xc, xs, wc, ws), y


def _ref_nvfp4(x, w, b):
    xq = o.nvfp4_quantize(x, x.float().abs().max())
    wq = o.nvfp4_quantize(w, w.float().abs().max())
    y = o.nvfp4_dequantize(*xq).cuda() @ o.nvfp4_dequantize(*wq).cuda().t()
    if b is not None:
        y = y + b.float().cuda()
    return xq, wq, y


@pytest.fixture(autouse=True, scope="module")
def _no_tf32():
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old


FP8_SHAPES = [(128, 128, 128), (128, 256, 512), (1, 4096, 4096), (16, 4096, 4096), (128, 14336, 4096),
              (200, 384, 1040), (77, 520, 144), (256, 264, 4096), (2048, 4096, 4096), (300, 4096, 14336)]


@pytest.mark.parametrize("bn", [128, 256, 512])
@pytest.mark.parametrize("M,N,K", FP8_SHAPES)
def test_fp8_gemm(capi, M, N, K, bn):
    x, w, b = _inputs(M, N, K, seed=2 + M + N + K)
    (xc, xs, wc, ws), ref = _ref_fp8(x, w, b)
    out = capi.fp8_gemm(xc.cuda(), xs.reshape(-1).cuda(), wc.cuda(), ws.reshape(-1).cuda(), b.cuda(), tile_n=bn)
    torch.cuda.synchronize()
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    assert o.rel_l2(out.float(), ref) <= TOL


SMALL_M = [(1, 4096, 4096), (16, 4096, 4096), (128, 4096, 14336), (64, 8192, 8192), (5, 520, 1040), (100, 384, 256), (33, 136, 4096)]


@pytest.mark.parametrize("force", [0, 128, 1001, 1002, 1004, 1008])
@pytest.mark.parametrize("M,N,K", SMALL_M)
def test_small_m_split_k(capi, M, N, K, force):
    """Decode-sized problems: swapped operands, K split over a CTA cluster, partials summed through
    distributed shared memory; every forced cluster size, the automatic choice, and the
    persistent 128-wide kernel on the same inputs."""
    if force > 1000 and (K + 127) // 128 < force - 1000:
        pytest.skip("fewer K tiles than splits")
    x, w, b = _inputs(M, N, K, seed=7 + M + N + K)
    (xc, xs, wc, ws), ref = _ref_fp8(x, w, b)
    out = capi.fp8_gemm(xc.cuda(), xs.reshape(-1).cuda(), wc.cuda(), ws.reshape(-1).cuda(), b.cuda(), tile_n=force)
    torch.cuda.synchronize()
    assert o.rel_l2(out.float(), ref) <= TOL
    if K % 32 == 0:
        xq, wq, ref4 = _ref_nvfp4(x, w, b)
        with capi.gemm_config(tile_n=force):           # the same selection through the per-thread default
            out = capi.nvfp4_gemm(xq[0].cuda(), o.swizzle_scales(xq[1]).cuda(), xq[2].cuda(),
                                  wq[0].cuda(), o.swizzle_scales(wq[1]).cuda(), wq[2].cuda(), b.cuda())
        torch.cuda.synchronize()
        assert o.rel_l2(out.float(), ref4) <= TOL


def test_fp8_gemm_per_tensor_scales_no_bias(capi):
    x, w, _ = _inputs(256, 512, 1024, seed=9, bias=False)
    xa, wa = x.float().abs().max(), w.float().abs().max()
    xc, xs = o.fp8_quantize(x, xa)
    wc, ws = o.fp8_quantize(w, wa)
    ref = o.fp8_dequantize(xc, xs).cuda() @ o.fp8_dequantize(wc, ws).cuda().t()
    out = capi.fp8_gemm(xc.cuda(), xs.reshape(1).cuda(), wc.cuda(), ws.reshape(1).cuda(), None)
    assert o.rel_l2(out.float(), ref) <= TOL


def test_fp8_gemm_exact_small_integers(capi):
    """Codes that are small integers with unit scales: every product and partial sum is exact in
    fp32 and representable in bf16, so the result must equal the integer matmul exactly."""
    g = torch.Generator().manual_seed(5)
    M, N, K = 256, 384, 256
    a = torch.randint(-2, 3, (M, K), generator=g).float()
    bm = torch.randint(-2, 3, (N, K), generator=g).float()
    ac, bc = o.e4m3_encode(a), o.e4m3_encode(bm)
    out = capi.fp8_gemm(ac.cuda(), torch.ones(1, device="cuda"), bc.cuda(), torch.ones(1, device="cuda"), None)
    assert torch.equal(out.float().cpu(), a @ bm.t())


NVFP4_SHAPES = [(128, 128, 256), (128, 256, 512), (16, 4096, 4096), (200, 384, 1056), (77, 520, 160),
                (256, 6144, 4096), (2048, 4096, 4096), (130, 4096, 14336)]


@pytest.mark.parametrize("bn", [128, 256, 512])
@pytest.mark.parametrize("M,N,K", NVFP4_SHAPES)
def test_nvfp4_gemm(capi, M, N, K, bn):
    x, w, b = _inputs(M, N, K, seed=3 + M + N + K)
    xq, wq, ref = _ref_nvfp4(x, w, b)
    out = capi.nvfp4_gemm(xq[0].cuda(), o.swizzle_scales(xq[1]).cuda(), xq[2].cuda(),
                          wq[0].cuda(), o.swizzle_scales(wq[1]).cuda(), wq[2].cuda(), b.cuda(), tile_n=bn)
    torch.cuda.synchronize()
    assert o.rel_l2(out.float(), ref) <= TOL


# ---------------------------------------------------------------- the M = 8192 shapes of the sweep
BIG = [(8192, 8192, 8192), (8192, 14336, 4096), (8192, 4096, 14336)]


@pytest.mark.parametrize("bn", [0, 128, 256])
@pytest.mark.parametrize("M,N,K", BIG[:2])
def test_fp8_gemm_m8192(capi, M, N, K, bn):
    """Many rounds of tiles per SM (pair): 0 = the automatic choice (CTA-pair kernel), 128 / 256 =
    the single-CTA kernel."""
    x, w, b = _inputs(M, N, K, seed=2 + M + N + K)
    (xc, xs, wc, ws), ref = _ref_fp8(x, w, b)
    out = capi.fp8_gemm(xc.cuda(), xs.reshape(-1).cuda(), wc.cuda(), ws.reshape(-1).cuda(), b.cuda(), tile_n=bn)
    torch.cuda.synchronize()
    assert o.rel_l2(out.float(), ref) <= TOL
    # no row or column block may be off on its own: the tolerance holds per 512 x 512 block too
    d, r = (out.float() - ref), ref
    blk = lambda t: t.view(M // 512, 512, N // 512, 512).pow(2).sum(dim=(1, 3)).sqrt()  # noqa: E731
    assert float((blk(d) / blk(r)).max()) <= 2 * TOL


@pytest.mark.parametrize("bn", [0, 512])
@pytest.mark.parametrize("M,N,K", BIG)
def test_nvfp4_gemm_m8192(capi, M, N, K, bn):
    x, w, b = _inputs(M, N, K, seed=3 + M + N + K)
    xq, wq, ref = _ref_nvfp4(x, w, b)
    out = capi.nvfp4_gemm(xq[0].cuda(), o.swizzle_scales(xq[1]).cuda(), xq[2].cuda(),
                          wq[0].cuda(), o.swizzle_scales(wq[1]).cuda(), wq[2].cuda(), b.cuda(), tile_n=bn)
    torch.cuda.synchronize()
    assert o.rel_l2(out.float(), ref) <= TOL
    d, r = (out.float() - ref), ref
    blk = lambda t: t.view(M // 512, 512, N // 512, 512).pow(2).sum(dim=(1, 3)).sqrt()  # noqa: E731
    assert float((blk(d) / blk(r)).max()) <= 2 * TOL


def test_config1_fp8_per_tensor_linear_full_size(capi):
    """FP8 per-tensor Q/DQ linear at the configuration's full size: x bf16 [16, 4096] ~ N(0,1),
    W bf16 [4096, 4096] ~ N(0, 0.02), seed 0, scales amax / 448 per tensor; the device path
    (amax, quantize, GEMM) against the oracle's linear on the same tensors."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(16, 4096, generator=g).bfloat16()
    w = (torch.randn(4096, 4096, generator=g) * 0.02).bfloat16()
    xa, wa = x.float().abs().max(), w.float().abs().max()
    ref = o.fp8_linear_ref(x, w, None, xa, wa)
    xd, wd = x.cuda(), w.cuda()
    ax, aw = capi.amax(xd), capi.amax(wd)
    assert ax.item() == xa.item() and aw.item() == wa.item()
    xc, xs = capi.fp8_quantize(xd, ax)
    wc, ws = capi.fp8_quantize(wd, aw)
    assert torch.equal(xc.cpu(), o.fp8_quantize(x, xa)[0]) and torch.equal(wc.cpu(), o.fp8_quantize(w, wa)[0])
    for tile in (0, 128, 1001, 1004):
        y = capi.fp8_gemm(xc, xs, wc, ws, None, tile_n=tile)
        assert y.shape == (16, 4096) and o.rel_l2(y.float().cpu(), ref) <= TOL


# ---------------------------------------------------------------- exact cases
# Sparse small integers: every product and every partial sum is an integer far below 2^24, so fp32
# accumulation is exact in any order, and the totals stay within +-256, where bf16 holds every
# integer.  The device result must EQUAL the integer matmul: a dropped or doubled 32/64-element
# K sub-block, a tile written to the wrong place or a mis-indexed scale shows as an integer error
# that no rel-L2 tolerance can absorb.
def _sparse_ints(rows, cols, g, density=1 / 8, top=2):
    v = torch.randint(1, top + 1, (rows, cols), generator=g).float()
    v = v * (torch.randint(0, 2, (rows, cols), generator=g).float() * 2 - 1)
    return v * (torch.rand(rows, cols, generator=g) < density)


EXACT_FP8 = [(0, 256, 384, 256), (128, 640, 640, 4096), (256, 640, 768, 4096), (512, 4096, 2560, 4096), (0, 2304, 4352, 8192),
             (1001, 64, 1024, 4096), (1002, 64, 1024, 4096), (1004, 128, 1152, 4096), (1008, 16, 1024, 8192), (0, 64, 8192, 8192)]


@pytest.mark.parametrize("tile,M,N,K", EXACT_FP8)
def test_fp8_gemm_exact_sparse_integers(capi, tile, M, N, K):
    """Every FP8 kernel: single-CTA 128 / 256 wide, the CTA-pair kernel with more than two tile
    rounds per SM pair (160 and 153 tiles of 256 x 256 on 74 pairs), the small-M kernel at every
    cluster size.  Row and column scales are powers of two (exact), so scale indexing is checked
    with the same equality."""
    g = torch.Generator().manual_seed(5 + tile + M + N + K)
    a, bm = _sparse_ints(M, K, g), _sparse_ints(N, K, g)
    sa = torch.tensor([0.5, 1.0, 2.0])[torch.randint(0, 3, (M,), generator=g)]
    sb = torch.tensor([0.5, 1.0, 2.0])[torch.randint(0, 3, (N,), generator=g)]
    raw = a.cuda() @ bm.cuda().t()
    assert float(raw.abs().max()) <= 256               # integers bf16 holds exactly; the power-of-two scales keep that
    ref = raw * sa.cuda()[:, None] * sb.cuda()[None, :]
    out = capi.fp8_gemm(o.e4m3_encode(a).cuda(), sa.cuda(), o.e4m3_encode(bm).cuda(), sb.cuda(), None, tile_n=tile)
    torch.cuda.synchronize()
    bad = (out.float() != ref).nonzero()
    assert bad.numel() == 0, f"{bad.shape[0]} wrong elements, first at {bad[0].tolist()}"


EXACT_NVFP4 = [(128, 256, 384, 4096), (256, 640, 768, 4096), (512, 1024, 1280, 4096), (0, 2304, 4352, 8192), (0, 384, 640, 4416),
               (1001, 64, 1024, 4096), (1004, 128, 1152, 4096), (1008, 16, 1024, 8192)]


@pytest.mark.parametrize("tile,M,N,K", EXACT_NVFP4)
def test_nvfp4_gemm_exact_sparse_integers(capi, tile, M, N, K):
    """NVFP4 kernels with hand-built operands: E2M1 codes 0 / +-1 / +-2, E4M3 block scales 1 or 2
    chosen per 16-element block, global scales 1 and 0.5.  The dequantized operands are small
    integers, so the result is exact: a scale atom read from the wrong row, column tile or K block
    changes integers.  K = 4416 ends in a partial 256-element K tile."""
    g = torch.Generator().manual_seed(9 + tile + M + N + K)

    def operand(rows):
        vals = _sparse_ints(rows, K, g, density=1 / 16)                       # in {0, +-1, +-2}
        codes = o.e2m1_encode(vals)
        blk = torch.tensor([1.0, 2.0])[torch.randint(0, 2, (rows, K // 16), generator=g)]
        return vals.view(rows, K // 16, 16) * blk[..., None], o.pack_e2m1(codes), o.e4m3_encode(blk)

    av, ac, asf = operand(M)
    bv, bc, bsf = operand(N)
    ga, gb = torch.tensor(1.0), torch.tensor(0.5)
    # the oracle's dequantize reproduces the hand-built values
    assert torch.equal(o.nvfp4_dequantize(ac, asf, ga), av.view(M, K))
    raw = av.view(M, K).cuda() @ bv.view(N, K).cuda().t()
    assert float(raw.abs().max()) <= 256
    ref = raw * 0.5
    out = capi.nvfp4_gemm(ac.cuda(), o.swizzle_scales(asf).cuda(), ga.cuda(), bc.cuda(), o.swizzle_scales(bsf).cuda(), gb.cuda(),
                          None, tile_n=tile)
    torch.cuda.synchronize()
    bad = (out.float() != ref).nonzero()
    assert bad.numel() == 0, f"{bad.shape[0]} wrong elements, first at {bad[0].tolist()}"


def test_golden_linear(b200):
    c = np.load(G / "cases.npz")
    x = torch.from_numpy(c["lin_x"]).bfloat16().cuda()
    w = torch.from_numpy(c["lin_w"]).bfloat16().cuda()
    b = torch.from_numpy(c["lin_b"]).bfloat16().cuda()
    y = b200.Fp8Linear.from_float(w, b)(x)
    assert o.rel_l2(y.float().cpu(), torch.from_numpy(c["lin_fp8"])) <= TOL
    y = b200.Fp8Linear.from_float(w, b, per_channel=False, input_amax=x.float().abs().max())(x)
    assert o.rel_l2(y.float().cpu(), torch.from_numpy(c["lin_fp8_tensor"])) <= TOL
    y = b200.Nvfp4Linear.from_float(w, b)(x)
    assert o.rel_l2(y.float().cpu(), torch.from_numpy(c["lin_nvfp4"])) <= TOL


@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
def test_fused_linear_matches_unfused_qdq_graph(b200, mode):
    """The fused layer against the eager Q/DQ graph the reference would hand to TensorRT
    (fake-quant ops + bf16 linear); 3-D input, bias."""
    x, w, b = _inputs(96, 512, 1024, seed=21)
    x = x.view(4, 24, 1024).cuda()
    w, b = w.cuda(), b.cuda()
    if mode == "fp8":
        fused = b200.Fp8Linear.from_float(w, b, per_channel=False, input_amax=b200.capi.amax(x))(x)
    else:
        fused = b200.Nvfp4Linear.from_float(w, b, input_amax=b200.capi.amax(x))(x)
    unfused = b200.QuantizedLinear(w, b, mode, input_amax=b200.capi.amax(x))(x)
    assert fused.shape == (4, 24, 512)
    assert o.rel_l2(fused.float(), unfused.float()) <= TOL


def test_torch_library_gemm_ops(b200):
    x, w, b = _inputs(64, 256, 512, seed=33)
    (xc, xs, wc, ws), ref = _ref_fp8(x, w, b)
    codes, scales = torch.ops.tensorrt.b200_fp8_quantize(x.cuda(), None)
    assert torch.equal(codes.cpu(), xc)
    out = torch.ops.tensorrt.b200_fp8_gemm_bias(codes, scales, wc.cuda(), ws.reshape(-1).cuda(), b.cuda())
    assert o.rel_l2(out.float(), ref) <= TOL
    nob = torch.ops.tensorrt.b200_fp8_gemm(codes, scales, wc.cuda(), ws.reshape(-1).cuda())
    assert o.rel_l2(nob.float(), ref - b.float().cuda()) <= TOL
    one = torch.ops.tensorrt.b200_fp8_linear_bias(x.cuda(), torch.empty(0, device="cuda"), wc.cuda(), ws.reshape(-1).cuda(), b.cuda())
    assert torch.equal(one, out)                       # empty amax = per-token abs-max measured by the kernel
    xq, wq, ref = _ref_nvfp4(x, w, b)
    c, s, g = torch.ops.tensorrt.b200_nvfp4_quantize(x.cuda(), x.float().abs().max().cuda())
    assert torch.equal(c.cpu(), xq[0])
    wc4, ws4, wg4 = torch.ops.tensorrt.b200_nvfp4_quantize(w.cuda(), w.float().abs().max().cuda())
    out = torch.ops.tensorrt.b200_nvfp4_gemm_bias(c, s, g, wc4, ws4, wg4, b.cuda())
    assert o.rel_l2(out.float(), ref) <= TOL
    one = torch.ops.tensorrt.b200_nvfp4_linear_bias(x.cuda(), x.float().abs().max().cuda(), wc4, ws4, wg4, b.cuda())
    assert torch.equal(one, out)
    half = torch.ops.tensorrt.b200_nvfp4_linear(x.half().cuda(), x.float().abs().max().cuda(), wc4, ws4, wg4)
    assert half.dtype == torch.float16 and o.rel_l2(half.float(), ref - b.float().cuda()) <= TOL


@pytest.mark.gpu
@pytest.mark.parametrize("M,F,K,with_bias", [(256, 128, 128, False), (300, 256, 512, True), (2048, 1024, 1024, False),
                                             (4096, 3584, 2048, True), (8192, 1792, 4096, False)])
def test_gate_up_gemm_with_fused_activation_is_bit_identical(b200, M, F, K, with_bias):
    """b200q_fp8_gemm_silu_mul (gate rows then up rows in one weight, activation in the GEMM epilogue)
    against b200q_fp8_gemm + b200q_silu_mul on the same operands: the same bits, with a ragged last
    row tile, several tile rounds per SM pair, per-channel weight scales and a bias; and against the
    oracle's linear + silu * up."""
    capi = b200.capi
    g = torch.Generator().manual_seed(M + F + K)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(2 * F, K, generator=g) * 0.05).bfloat16()
    bias = (torch.randn(2 * F, generator=g) * 0.1).bfloat16() if with_bias else None
    xq = capi.fp8_quantize(x.cuda(), None)
    wq = capi.fp8_quantize(w.cuda(), capi.row_amax(w.cuda()))
    bd = None if bias is None else bias.cuda()
    fused = capi.fp8_gemm_silu_mul(xq[0], xq[1], wq[0], wq[1], bd)
    ref = capi.silu_mul(capi.fp8_gemm(xq[0], xq[1], wq[0], wq[1], bd))
    assert fused.shape == (M, F) and torch.equal(fused, ref)
    assert capi.device_status() == 0
    y = o.fp8_linear_ref(x, w, bias).float()
    want = torch.nn.functional.silu(y[:, :F].bfloat16().float()) * y[:, F:].bfloat16().float()
    assert o.rel_l2(fused.float().cpu(), want) < 1e-2
    with pytest.raises(ValueError):
        capi.fp8_gemm_silu_mul(xq[0], xq[1], wq[0][:2 * F - 128], wq[1][:2 * F - 128])     # F not a multiple of 128
    # ... and with the static per-tensor quantizer of the activation in the epilogue as well: the codes and the scale
    # of quantizing the bf16 result, for an amax above the data and one below it (the clamp)
    for amax in (fused.float().abs().max() * 1.25, fused.float().abs().max() * 0.3, torch.zeros((), device="cuda")):
        codes, scale = capi.fp8_gemm_silu_mul_quantize(xq[0], xq[1], wq[0], wq[1], amax.reshape(1), bd)
        c_ref, s_ref = capi.fp8_quantize(fused, amax.reshape(1))
        assert torch.equal(codes, c_ref) and torch.equal(scale.reshape(-1), s_ref.reshape(-1))
    assert capi.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [8, 300])
@pytest.mark.parametrize("static", [False, True])
def test_gated_mlp_module(b200, tokens, static):
    """Fp8GatedMlp (stacked gate/up weight, activation and, with a static amax, its quantizer in the GEMM
    epilogue) against the same MLP built from three Fp8Linear modules and this library's silu * up kernel (the
    same bits), and against the oracle's linears with an fp32 activation (close)."""
    capi = b200.capi
    g = torch.Generator().manual_seed(tokens)
    hdim, f = 256, 384
    x = torch.randn(2, tokens // 2, hdim, generator=g).bfloat16().cuda()
    wg, wu = ((torch.randn(f, hdim, generator=g) * 0.06).bfloat16().cuda() for _ in range(2))
    wd = (torch.randn(hdim, f, generator=g) * 0.05).bfloat16().cuda()
    in_amax = x.float().abs().max().reshape(1) if static else None
    gate, up, down = (b200.Fp8Linear.from_float(w, input_amax=in_amax) for w in (wg, wu, wd))
    act = capi.silu_mul(torch.cat([gate(x), up(x)], dim=-1))
    act_amax = (act.float().abs().max() * 0.9).reshape(1) if static else None
    down.input_amax = act_amax
    ref = down(act)
    mlp = b200.Fp8GatedMlp.from_float(wg, wu, wd, input_amax=in_amax, act_amax=act_amax)
    y = mlp(x)
    assert y.shape == x.shape and torch.equal(y, ref)
    assert capi.device_status() == 0
    yo = o.fp8_linear_ref(x.cpu().reshape(-1, hdim), torch.cat([wg, wu]).cpu()).bfloat16().float()
    want = o.fp8_linear_ref((torch.nn.functional.silu(yo[:, :f]) * yo[:, f:]).bfloat16(), wd.cpu())
    if not static:
        assert o.rel_l2(y.float().cpu().reshape(-1, hdim), want.float()) < 2e-2
    with pytest.raises(ValueError):
        b200.Fp8GatedMlp.from_float(wg[:192], wu[:192], wd[:, :192])        # 192 is not a multiple of 128
