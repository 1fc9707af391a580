"""CPU tests of the oracle: number formats, golden fixtures, properties."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as o

G = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def formats():
    return np.load(G / "formats.npz")


@pytest.fixture(scope="module")
def cases():
    return np.load(G / "cases.npz")


def test_e4m3_decode_table_matches_torch_dtype(formats):
    ours = o.e4m3_decode_table()
    ref = formats["e4m3"]
    assert np.array_equal(np.isnan(ours), np.isnan(ref))
    assert np.array_equal(ours[~np.isnan(ours)], ref[~np.isnan(ref)])
    assert ours[0x7E] == 448.0 and ours[0x01] == 2.0 ** -9


def test_e4m3_encoders_agree_on_every_fp16_value():
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16).float()
    bits = bits[torch.isfinite(bits)]
    assert np.array_equal(o.e4m3_encode(bits).numpy(), o.e4m3_encode_np(bits.numpy()))


def test_e4m3_round_to_nearest_even_and_saturation():
    x = torch.tensor([17.0, 19.0, 2.0 ** -10, 1.5 * 2.0 ** -10, 448.0, 464.0, 1e9, -1e9, -0.0])
    codes = o.e4m3_encode(x)
    dec = o.e4m3_decode(codes)
    assert dec.tolist()[:4] == [16.0, 20.0, 0.0, 2.0 ** -9]
    assert dec[4:8].tolist() == [448.0, 448.0, 448.0, -448.0]
    assert codes[-1].item() == 0x80


def test_e2m1_ties_and_golden(formats):
    got = o.e2m1_encode(torch.from_numpy(formats["probe_e2m1"])).numpy()
    assert np.array_equal(got, formats["code_e2m1"])
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert o.e2m1_decode(o.e2m1_encode(ties)).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]
    assert np.array_equal(o.e2m1_decode(torch.arange(16, dtype=torch.uint8)).numpy(), formats["e2m1"])
    # decode(encode(v)) is the identity on the grid, sign bit included
    grid = torch.from_numpy(formats["e2m1"])
    assert torch.equal(o.e2m1_encode(grid), torch.arange(16, dtype=torch.uint8))


def test_pack_is_low_nibble_first():
    codes = torch.tensor([[1, 2, 3, 15]], dtype=torch.uint8)
    packed = o.pack_e2m1(codes)
    assert packed.tolist() == [[0x21, 0xF3]]
    assert torch.equal(o.unpack_e2m1(packed), codes)


@pytest.mark.parametrize("rows,cols", [(1, 1), (128, 4), (129, 5), (300, 37), (512, 512)])
def test_swizzle_roundtrip_and_layout(rows, cols):
    s = torch.randint(0, 255, (rows, cols), dtype=torch.uint8)
    buf = o.swizzle_scales(s)
    assert buf.numel() == o.swizzled_scale_bytes(rows, cols * 16)
    assert torch.equal(o.unswizzle_scales(buf, rows, cols), s)
    ct = (cols + 3) // 4
    for r, c in [(0, 0), (rows - 1, cols - 1), (rows // 2, cols // 2)]:
        off = ((r // 128) * ct + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
        assert buf[off] == s[r, c]


@pytest.mark.parametrize("name,dtype", [("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)])
def test_golden_cases(cases, name, dtype):
    x = torch.from_numpy(cases[f"{name}_x"]).to(dtype)
    amax_t = x.float().abs().max()
    c, s = o.fp8_quantize(x, amax_t)
    assert np.array_equal(c.numpy(), cases[f"{name}_fp8_tensor_codes"])
    assert np.array_equal(s.numpy(), cases[f"{name}_fp8_tensor_scale"])
    c, s = o.fp8_quantize(x, o.row_amax(x))
    assert np.array_equal(c.numpy(), cases[f"{name}_fp8_row_codes"])
    assert np.array_equal(s.numpy(), cases[f"{name}_fp8_row_scale"])
    p, sc, g = o.nvfp4_quantize(x, amax_t)
    assert np.array_equal(p.numpy(), cases[f"{name}_nvfp4_codes"])
    assert np.array_equal(sc.numpy(), cases[f"{name}_nvfp4_scales"])
    assert np.array_equal(o.swizzle_scales(sc).numpy(), cases[f"{name}_nvfp4_scales_swizzled"])
    assert g.item() == cases[f"{name}_nvfp4_global"].item()
    assert np.array_equal(o.nvfp4_fake_quant(x, amax_t).float().numpy(), cases[f"{name}_nvfp4_fake"])


def test_zero_rows_and_blocks(cases):
    x = torch.from_numpy(cases["bf16_x"]).bfloat16()
    c, s = o.fp8_quantize(x, o.row_amax(x))
    assert s[5].item() == 1.0 and int(c[5].max()) == 0          # all-zero row: scale 1, codes 0
    p, sc, _ = o.nvfp4_quantize(x, x.float().abs().max())
    assert int(sc[5].max()) == 0 and int(p[5].max()) == 0
    assert int(sc[9, 1]) == 0 and int(p[9, 8:16].max()) == 0       # block whose stored scale rounds to 0
    assert int(p[7, :8].max()) == 0                                 # -0.0 inputs in a zero-scale block give code 0


def test_fake_quant_is_idempotent():
    g = torch.Generator().manual_seed(7)
    x = torch.randn(64, 128, generator=g).bfloat16()
    a = o.row_amax(x)
    y = o.fp8_fake_quant(x, a)
    assert torch.equal(o.fp8_fake_quant(y, a), y)


def test_op_level_argument_checks():
    x = torch.randn(4, 32)
    with pytest.raises(ValueError):
        o.quantize_op(x, torch.tensor(1.0), 8, 0, False, False)
    with pytest.raises(ValueError):
        o.quantize_op(x.to(torch.int32), torch.tensor(1.0))
    with pytest.raises(ValueError):
        o.dynamic_block_quantize_op(torch.randn(4, 24), 16, torch.tensor(1.0))
    y = o.dynamic_block_quantize_op(torch.randn(2, 3, 4, 32), 16, torch.tensor(3.0))
    assert y.shape == (2, 3, 4, 32)


def test_global_scale_formula():
    assert o.nvfp4_global_scale(torch.tensor(0.0)).item() == 1.0
    a = torch.tensor(5.0)
    assert o.nvfp4_global_scale(a).item() == ((a / 6) / 448).item()
    assert o.fp8_scale(torch.tensor([0.0, 448.0])).tolist() == [1.0, 1.0]


def test_linear_golden_and_tolerance(cases):
    x = torch.from_numpy(cases["lin_x"]).bfloat16()
    w = torch.from_numpy(cases["lin_w"]).bfloat16()
    b = torch.from_numpy(cases["lin_b"]).bfloat16()
    assert np.array_equal(o.fp8_linear_ref(x, w, b).numpy(), cases["lin_fp8"])
    assert np.array_equal(o.nvfp4_linear_ref(x, w, b).numpy(), cases["lin_nvfp4"])
    exact = x.float() @ w.float().t() + b.float()
    assert o.rel_l2(torch.from_numpy(cases["lin_fp8"]), exact) < 0.05
    assert o.rel_l2(torch.from_numpy(cases["lin_nvfp4"]), exact) < 0.2


def test_config1_fp8_per_tensor_linear_cpu():
    """FP8 per-tensor Q/DQ linear on CPU: x bf16 [16, 4096] ~ N(0,1), W bf16 [4096, 4096] ~ N(0, 0.02), seed 0."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(16, 4096, generator=g).bfloat16()
    w = (torch.randn(4096, 4096, generator=g) * 0.02).bfloat16()
    xq = o.quantize_op(x, x.float().abs().max())
    wq = o.quantize_op(w, w.float().abs().max())
    y = (xq.float() @ wq.float().t()).bfloat16()
    assert y.shape == (16, 4096)
    assert o.rel_l2(y.float(), x.float() @ w.float().t()) < 0.06
    # real-quant route gives the same numbers up to the bf16 rounding of the fake-quant tensors
    y2 = o.fp8_linear_ref(x, w, None, x.float().abs().max(), w.float().abs().max())
    assert o.rel_l2(y2, y.float()) < 0.01


def test_all_reduce_known_answer():
    for world in (1, 2, 4, 8):
        parts = [torch.full((1, 4), float(r + 1)) for r in range(world)]
        assert torch.allclose(o.all_reduce_ref(parts), torch.full((1, 4), world * (world + 1) / 2), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
def test_tensor_parallel_layer_matches_single_rank(mode):
    g = torch.Generator().manual_seed(4)
    hid, nq, nkv, hd, ffn = 256, 4, 2, 64, 512
    layer = {
        "norm1": torch.ones(hid), "norm2": torch.ones(hid),
        "wqkv": (torch.randn((nq + 2 * nkv) * hd, hid, generator=g) * 0.02).bfloat16(),
        "wo": (torch.randn(hid, nq * hd, generator=g) * 0.02).bfloat16(),
        "wgu": (torch.randn(2 * ffn, hid, generator=g) * 0.02).bfloat16(),
        "wdown": (torch.randn(hid, ffn, generator=g) * 0.02).bfloat16(),
    }
    h = torch.randn(2, 8, hid, generator=g).bfloat16()
    y1 = o.decoder_layer_ref(h, layer, nq, nkv, hd, mode, world=1)
    y2 = o.decoder_layer_ref(h, layer, nq, nkv, hd, mode, world=2)
    assert y1.shape == h.shape
    assert o.rel_l2(y2.float(), y1.float()) < (2e-2 if mode == "fp8" else 8e-2)


def _close_in_bf16(a: torch.Tensor, b: np.ndarray) -> bool:
    """Equal up to one unit in the last place of bf16 (fp32 sums inside may be ordered differently on another CPU)."""
    b = torch.from_numpy(b)
    return bool(((a.float() - b).abs() <= 2.0 ** -7 * torch.maximum(a.float().abs(), b.abs()) + 1e-6).all())


def test_golden_attention_all_reduce_and_decoder_layer():
    """Fixtures of the layer-level restatements (tests/golden/layers.npz, generator beside it): FP8 attention with
    GQA, the lower-right causal mask and a short query block; the fp32-sum all-reduce; a decoder layer in both
    modes, as 1 and 2 tensor-parallel ranks, with the identity and the FP8-attention core."""
    z = np.load(G / "layers.npz")
    q, k, v = (torch.from_numpy(z[f"sdpa_{n}"]).half() for n in "qkv")
    am = torch.tensor(3.5)
    assert _close_in_bf16(o.fp8_sdpa_ref(q, k, v, am, am, am), z["sdpa_full"])
    assert _close_in_bf16(o.fp8_sdpa_ref(q, k, v, am, am, am, is_causal=True), z["sdpa_causal"])
    assert _close_in_bf16(o.fp8_sdpa_ref(q[:, :, -8:], k, v, am, am, am, is_causal=True), z["sdpa_causal_short_q"])
    assert not np.array_equal(z["sdpa_full"], z["sdpa_causal"])
    # the last 8 queries of the full causal problem see the same keys as the short query block aligned to the end
    assert np.allclose(z["sdpa_causal"][:, :, -8:], z["sdpa_causal_short_q"], atol=1e-3)
    parts = [t.bfloat16() for t in torch.from_numpy(z["ar_parts"])]
    assert np.array_equal(o.all_reduce_ref(parts, torch.bfloat16).float().numpy(), z["ar_sum"])
    layer = {key: torch.from_numpy(z[f"layer_{key}"]).bfloat16() for key in ("norm1", "norm2", "wqkv", "wo", "wgu", "wdown")}
    h = torch.from_numpy(z["layer_h"]).bfloat16()
    for mode in ("fp8", "nvfp4"):
        for world in (1, 2):
            assert _close_in_bf16(o.decoder_layer_ref(h, layer, 4, 2, 16, mode, world=world), z[f"layer_{mode}_w{world}"]), (mode, world)
    assert _close_in_bf16(o.decoder_layer_ref(h, layer, 4, 2, 16, "fp8", world=2, attention="fp8_sdpa", seq_len=8), z["layer_fp8_sdpa_w2"])
