"""GPU parity of the quantize kernels, called through the C ABI, against the CPU oracle:
bit-exact codes, block scales, global scales and fake-quant outputs."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as o

pytestmark = pytest.mark.gpu
G = Path(__file__).parent / "golden"
DTYPES = [("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)]


@pytest.fixture(scope="module")
def capi(b200):
    return b200.capi


@pytest.fixture(scope="module")
def cases():
    return np.load(G / "cases.npz")


def _cuda(t):
    return t.cuda()


def _mismatch(a: torch.Tensor, b: torch.Tensor) -> int:
    return int((a.cpu() != b.cpu()).sum())


@pytest.mark.parametrize("name,dtype", DTYPES)
def test_golden_fp8(capi, cases, name, dtype):
    x = torch.from_numpy(cases[f"{name}_x"]).to(dtype)
    xd = _cuda(x)
    amax_t = x.float().abs().max()
    codes, scales = capi.fp8_quantize(xd, _cuda(amax_t))
    assert np.array_equal(codes.cpu().numpy(), cases[f"{name}_fp8_tensor_codes"])
    assert scales.cpu().numpy().reshape(()) == cases[f"{name}_fp8_tensor_scale"].reshape(())
    for amax in (_cuda(o.row_amax(x)), None):  # supplied per-row amax, then reduced in-kernel
        codes, scales = capi.fp8_quantize(xd, amax)
        assert np.array_equal(codes.cpu().numpy(), cases[f"{name}_fp8_row_codes"])
        assert np.array_equal(scales.cpu().numpy().reshape(-1, 1), cases[f"{name}_fp8_row_scale"])
    fake = capi.fp8_fake_quantize(xd, None)
    assert np.array_equal(fake.float().cpu().numpy(), cases[f"{name}_fp8_fake"])


@pytest.mark.parametrize("name,dtype", DTYPES)
def test_golden_nvfp4(capi, cases, name, dtype):
    x = torch.from_numpy(cases[f"{name}_x"]).to(dtype)
    xd = _cuda(x)
    amax_t = _cuda(x.float().abs().max())
    codes, sf, g = capi.nvfp4_quantize(xd, amax_t)
    assert np.array_equal(codes.cpu().numpy(), cases[f"{name}_nvfp4_codes"])
    assert np.array_equal(sf.cpu().numpy(), cases[f"{name}_nvfp4_scales_swizzled"])  # padding bytes included
    assert g.item() == cases[f"{name}_nvfp4_global"].item()
    fake = capi.nvfp4_fake_quantize(xd, amax_t)
    assert np.array_equal(fake.float().cpu().numpy(), cases[f"{name}_nvfp4_fake"])
    deq = capi.nvfp4_dequantize(codes, sf, g, dtype)
    assert np.array_equal(deq.float().cpu().numpy(), cases[f"{name}_nvfp4_fake"])


def test_golden_saturation(capi, cases):
    x = torch.from_numpy(cases["sat_x"]).bfloat16()
    small = torch.tensor(2.0)
    codes, _ = capi.fp8_quantize(_cuda(x), _cuda(small))
    assert np.array_equal(codes.cpu().numpy(), cases["sat_fp8_codes"])
    codes, sf, _ = capi.nvfp4_quantize(_cuda(x), _cuda(small))
    assert np.array_equal(codes.cpu().numpy(), cases["sat_nvfp4_codes"])
    assert np.array_equal(o.unswizzle_scales(sf.cpu(), 16, 4).numpy(), cases["sat_nvfp4_scales"])


def _make(rows, cols, dtype, seed, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    if outliers:
        x[torch.rand(rows, cols, generator=g) < 0.01] *= 50
    return x.to(dtype)


SHAPES = [(1, 16), (1, 4096), (3, 48), (16, 4096), (127, 2064), (129, 6144), (130, 14336), (33, 28672), (5, 40000 // 16 * 16)]


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_fp8_random_shapes(capi, rows, cols, dtype):
    x = _make(rows, cols, dtype, seed=rows * 7 + cols)
    xd = _cuda(x)
    ref_c, ref_s = o.fp8_quantize(x, o.row_amax(x))
    codes, scales = capi.fp8_quantize(xd, None)
    assert _mismatch(codes, ref_c) == 0
    assert torch.equal(scales.cpu().view(-1, 1), ref_s)
    amax_t = x.float().abs().max() * 0.5  # static amax below the true maximum: exercises the clamp
    ref_c, _ = o.fp8_quantize(x, amax_t)
    codes, _ = capi.fp8_quantize(xd, _cuda(amax_t))
    assert _mismatch(codes, ref_c) == 0
    assert torch.equal(capi.fp8_fake_quantize(xd, _cuda(amax_t)).cpu(), o.fp8_fake_quant(x, amax_t))
    assert torch.equal(capi.fp8_dequantize(codes, _cuda(o.fp8_scale(amax_t).reshape(1)), dtype).cpu(),
                       o.fp8_fake_quant(x, amax_t))


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_nvfp4_random_shapes(capi, rows, cols, dtype):
    x = _make(rows, cols, dtype, seed=rows * 11 + cols)
    xd = _cuda(x)
    for amax in (x.float().abs().max(), x.float().abs().max() * 0.25):
        ref_p, ref_s, ref_g = o.nvfp4_quantize(x, amax)
        codes, sf, g = capi.nvfp4_quantize(xd, _cuda(amax))
        assert g.item() == ref_g.item()
        assert torch.equal(sf.cpu(), o.swizzle_scales(ref_s)), "block scales / swizzled layout / zero padding"
        assert _mismatch(codes, ref_p) == 0
        assert torch.equal(capi.nvfp4_fake_quantize(xd, _cuda(amax)).cpu(), o.nvfp4_fake_quant(x, amax))


def test_amax_kernels(capi):
    for n in (1, 7, 8, 1000, 8192 * 33 + 5):
        for dtype in (torch.bfloat16, torch.float16, torch.float32):
            x = _make(1, n, dtype, seed=n)[0]
            assert capi.amax(_cuda(x)).item() == x.float().abs().max().item()
            assert capi.amax(_cuda(x)).item() == x.float().abs().max().item()  # workspace re-armed
    x = _make(257, 4104, torch.bfloat16, seed=5)
    assert torch.equal(capi.row_amax(_cuda(x)).cpu(), o.row_amax(x))
    # many 32-byte chunks per thread (the unrolled part of the kernel), then a 16-byte group and a
    # scalar tail; the maximum is planted in each region in turn, with both signs, and the same
    # again from a base pointer that is only 16-byte aligned (the narrow-load path)
    n = 1184 * 256 * 16 * 9 + 8 + 5
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        base = torch.rand(n + 8, dtype=torch.float32).to(dtype).cuda()
        for off in (0, 8 if dtype != torch.float32 else 4):
            x = base[off:off + n]
            assert x.data_ptr() % 32 == (0 if off == 0 else 16)
            for pos in (0, 12345, 1184 * 256 * 16 * 8 + 77, n - 14, n - 13, n - 1):
                for val in (3.0, -5.0):
                    keep = x[pos].item()
                    x[pos] = val
                    assert capi.amax(x).item() == abs(val), (dtype, off, pos)
                    x[pos] = keep
            assert capi.amax(x).item() == x.float().abs().max().item()


def test_special_values(capi):
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    x[1] = -0.0
    x[2, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[3, 0] = 448.0
    x[3, 1] = -1e-30
    for amax in (torch.tensor(6.0), torch.tensor(448.0), torch.tensor(0.0)):
        ref = o.nvfp4_quantize(x, amax)
        got = capi.nvfp4_quantize(_cuda(x), _cuda(amax))
        assert torch.equal(got[0].cpu(), ref[0]) and torch.equal(got[1].cpu(), o.swizzle_scales(ref[1]))
        ref_c, _ = o.fp8_quantize(x, amax)
        assert torch.equal(capi.fp8_quantize(_cuda(x), _cuda(amax))[0].cpu(), ref_c)
    ref_c, ref_s = o.fp8_quantize(x, o.row_amax(x))
    codes, scales = capi.fp8_quantize(_cuda(x), None)
    assert torch.equal(codes.cpu(), ref_c) and torch.equal(scales.cpu().view(-1, 1), ref_s)


def test_empty_inputs(capi):
    x = torch.empty(0, 64, dtype=torch.bfloat16, device="cuda")
    codes, scales = capi.fp8_quantize(x, None)
    assert codes.shape == (0, 64) and scales.numel() == 0
    codes, sf, g = capi.nvfp4_quantize(x, torch.tensor(1.0, device="cuda"))
    assert codes.shape == (0, 32) and sf.numel() == 0


def test_config2_nvfp4_full_size(capi):
    """bf16 [8192, 8192] ~ N(0,1) with 1% of elements x50, seed 1: a [1024, 8192] slab is compared
    bit for bit with the oracle; the full tensor through size-independent properties."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn(8192, 8192, generator=g)
    x[torch.rand(8192, 8192, generator=g) < 0.01] *= 50
    x = x.bfloat16()
    amax = x.float().abs().max()
    xd = _cuda(x)
    assert capi.amax(xd).item() == amax.item()
    codes, sf, gs = capi.nvfp4_quantize(xd, _cuda(amax))
    ref_p, ref_s, ref_g = o.nvfp4_quantize(x[3072:4096], amax)
    assert gs.item() == ref_g.item()
    assert torch.equal(codes[3072:4096].cpu(), ref_p)
    full_sf = o.unswizzle_scales(sf.cpu(), 8192, 512)
    assert torch.equal(full_sf[3072:4096], ref_s)
    # quantize(dequantize(q)) reproduces q exactly (idempotence), at full size, on the device
    deq = capi.nvfp4_dequantize(codes, sf, gs, torch.bfloat16)
    codes2, sf2, _ = capi.nvfp4_quantize(deq, _cuda(amax))
    assert torch.equal(codes2, codes) and torch.equal(sf2, sf)
    assert torch.equal(capi.nvfp4_fake_quantize(xd, _cuda(amax)), deq)
    # block scales never under-cover the block: |x| <= 6 * d * (1 + 2^-4) (E4M3 rounding slack)
    d = (o.e4m3_decode(full_sf) * gs.cpu()).repeat_interleave(16, dim=1)
    assert bool((x.float().abs() <= d * 6 * (1 + 2.0 ** -4) + 1e-30).all())


def test_ops_through_torch_library(b200):
    x = _make(6, 4096, torch.bfloat16, seed=3).view(2, 3, 4096)
    xd = _cuda(x)
    amax = x.float().abs().max()
    y = torch.ops.tensorrt.quantize_op(xd, _cuda(amax), 8, 4, False, False)
    assert torch.equal(y.cpu(), o.quantize_op(x, amax))
    y = torch.ops.tensorrt.quantize_op(xd, _cuda(o.row_amax(x)), 8, 4, False, False)
    assert torch.equal(y.cpu(), o.fp8_fake_quant(x.view(6, 4096), o.row_amax(x.view(6, 4096))).view(2, 3, 4096))
    y = torch.ops.tensorrt.dynamic_block_quantize_op(xd, 16, _cuda(amax), 4, 2, 8, 4)
    assert torch.equal(y.cpu(), o.dynamic_block_quantize_op(x, 16, amax))
    assert torch.ops.tensorrt.b200_amax(xd).item() == amax.item()
    with pytest.raises(ValueError, match="Supported types"):
        torch.ops.tensorrt.quantize_op(xd.to(torch.int32), _cuda(amax), 8, 4, False, False)
    with pytest.raises(ValueError, match="FP8"):
        torch.ops.tensorrt.quantize_op(xd, _cuda(amax), 8, 0, False, False)
    with pytest.raises(ValueError, match="multiple of the block size"):
        torch.ops.tensorrt.dynamic_block_quantize_op(xd[..., :24], 16, _cuda(amax), 4, 2, 8, 4)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(1184, 4096), (1200, 16384), (1300, 16400), (1190, 20480), (1185, 28672), (1186, 32768)])
def test_per_token_quantize_of_many_long_rows(capi, rows, cols):
    """Rows longer than 16384 elements, 8 or more per SM: the dynamic per-token bf16 quantize runs as persistent
    CTAs fed through a shared-memory ring; shorter rows keep one CTA per row.  Either way codes and scales are the
    oracle's bit for bit and equal to what slices of the same tensor give (an all-zero row included)."""
    x = _make(rows, cols, torch.bfloat16, seed=rows + cols)
    x[5] = 0
    xd = _cuda(x)
    codes, scales = capi.fp8_quantize(xd, None)
    ref_c, ref_s = o.fp8_quantize(x, o.row_amax(x))
    assert torch.equal(codes.cpu(), ref_c) and torch.equal(scales.cpu().reshape(-1), ref_s.reshape(-1))
    parts = [capi.fp8_quantize(xd[i:i + 500].contiguous(), None) for i in range(0, rows, 500)]
    assert torch.equal(codes, torch.cat([p[0] for p in parts])) and torch.equal(scales, torch.cat([p[1] for p in parts]))
    assert capi.device_status() == 0
