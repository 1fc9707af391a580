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
    capi.set_gemm_tile_n(0)
    yield
    capi.set_gemm_tile_n(0)
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
    capi.set_gemm_tile_n(bn)
    out = capi.fp8_gemm(xc.cuda(), xs.reshape(-1).cuda(), wc.cuda(), ws.reshape(-1).cuda(), b.cuda())
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
    capi.set_gemm_tile_n(force)
    out = capi.fp8_gemm(xc.cuda(), xs.reshape(-1).cuda(), wc.cuda(), ws.reshape(-1).cuda(), b.cuda())
    torch.cuda.synchronize()
    assert o.rel_l2(out.float(), ref) <= TOL
    if K % 32 == 0:
        xq, wq, ref4 = _ref_nvfp4(x, w, b)
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
    capi.set_gemm_tile_n(bn)
    out = capi.nvfp4_gemm(xq[0].cuda(), o.swizzle_scales(xq[1]).cuda(), xq[2].cuda(),
                          wq[0].cuda(), o.swizzle_scales(wq[1]).cuda(), wq[2].cuda(), b.cuda())
    torch.cuda.synchronize()
    assert o.rel_l2(out.float(), ref) <= TOL


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
    out = torch.ops.tensorrt.b200_fp8_gemm(codes, scales, wc.cuda(), ws.reshape(-1).cuda(), b.cuda())
    assert o.rel_l2(out.float(), ref) <= TOL
    xq, wq, ref = _ref_nvfp4(x, w, b)
    c, s, g = torch.ops.tensorrt.b200_nvfp4_quantize(x.cuda(), x.float().abs().max().cuda())
    assert torch.equal(c.cpu(), xq[0])
    wc4, ws4, wg4 = torch.ops.tensorrt.b200_nvfp4_quantize(w.cuda(), w.float().abs().max().cuda())
    out = torch.ops.tensorrt.b200_nvfp4_gemm(c, s, g, wc4, ws4, wg4, b.cuda())
    assert o.rel_l2(out.float(), ref) <= TOL
