"""FP8 attention (Q, K, V from `quantize_op(.., 8, 4, ..)`, softmax output quantized with scale 1/448)
against the oracle's restatement of the reference semantics
(py/torch_tensorrt/dynamo/lowering/passes/annotate_fp8_sdpa.py:34-76, conversion/impl/attention.py:272-337).
Tolerances: rel-L2 <= 1e-2 against the oracle (same quantization points; fp32 exponentials and summation
order differ), cosine similarity > 0.99 against plain fp32 attention, the bar of the reference's own test
(tests/py/dynamo/models/test_models_export.py:838-844)."""
import pytest
import torch

import oracle as o

TOL = 1e-2


def _qkv(B, Hq, Hkv, Sq, Sk, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, Sq, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, Sk, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, Sk, D, generator=g).to(dtype)
    return q, k, v


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().float()[None], b.flatten().float()[None]).item()


def test_oracle_on_the_reference_test_construction():
    """The reference's own FP8 MHA test: B, H, S, D = 1, 2, 32, 64, fp16 ~ N(0, 1), seed 0, amax 6.0 for all
    three quantizers, pass mark cosine > 0.99 against plain SDPA.  The oracle meets it on the CPU."""
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 2, 32, 64, dtype=torch.float16) for _ in range(3))
    amax = torch.tensor(6.0)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    out = o.fp8_sdpa_ref(q, k, v, amax, amax, amax)
    assert out.dtype == torch.float16 and _cos(out, ref) > 0.99
    # the softmax output really is on the E4M3 grid scaled by 1/448: quantizing twice changes nothing
    p = torch.softmax(torch.randn(4, 64), dim=-1)
    once = o.e4m3_decode(o.e4m3_encode(p * 448)) / 448
    assert torch.equal(o.e4m3_decode(o.e4m3_encode(once * 448)) / 448, once)
    # grouped-query heads and the lower-right causal mask against an explicit loop
    q, k, v = _qkv(1, 4, 2, 5, 9, 16, torch.float32, 3)
    out = o.fp8_sdpa_ref(q, k, v, amax, amax, amax, is_causal=True)
    qh, kh, vh = (o.fp8_dequantize(*o.fp8_quantize(t, amax)) for t in (q, k, v))
    for h in range(4):
        for i in range(5):
            vis = min(9, i + 9 - 5 + 1)
            s = (qh[0, h, i] @ kh[0, h // 2, :vis].t()) / 4.0
            p = o.e4m3_decode(o.e4m3_encode(torch.softmax(s, -1) * 448)) / 448
            assert torch.allclose(out[0, h, i], p @ vh[0, h // 2, :vis], atol=1e-5)


CASES = [
    # B, Hq, Hkv, Sq, Sk, D, dtype, causal
    (1, 2, 2, 32, 32, 64, torch.float16, False),          # the reference test's shape
    (2, 8, 2, 300, 300, 128, torch.bfloat16, False),      # grouped-query heads, ragged tiles
    (2, 8, 2, 300, 300, 128, torch.bfloat16, True),
    (1, 4, 4, 128, 128, 128, torch.bfloat16, True),
    (1, 4, 1, 16, 200, 64, torch.float16, True),          # fewer queries than keys: lower-right alignment
    (1, 2, 2, 257, 129, 32, torch.float32, False),
    (1, 2, 2, 200, 72, 48, torch.float32, True),          # more queries than keys: the first rows see nothing
    (1, 64, 8, 1024, 1024, 128, torch.bfloat16, True),    # one sequence of the 70B-shaped stack's attention
    (4, 2, 1, 1, 513, 128, torch.bfloat16, False),        # single-query decode step
]


@pytest.mark.gpu
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,D,dtype,causal", CASES)
def test_fp8_sdpa_matches_oracle(b200, B, Hq, Hkv, Sq, Sk, D, dtype, causal):
    q, k, v = _qkv(B, Hq, Hkv, Sq, Sk, D, dtype, seed=B + Hq + Sq + Sk + D)
    aq, ak, av = (t.float().abs().max() for t in (q, k, v))
    ref = o.fp8_sdpa_ref(q, k, v, aq, ak, av, is_causal=causal)
    out = b200.capi.fp8_sdpa(q.cuda(), k.cuda(), v.cuda(), aq.cuda(), ak.cuda(), av.cuda(), is_causal=causal)
    torch.cuda.synchronize()
    assert b200.capi.device_status() == 0
    assert out.shape == q.shape and out.dtype == dtype
    assert o.rel_l2(out.float().cpu(), ref.float()) <= TOL
    plain = torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float().repeat_interleave(Hq // Hkv, 1), v.float().repeat_interleave(Hq // Hkv, 1),
        attn_mask=(torch.ones(Sq, Sk, dtype=torch.bool).tril(Sk - Sq) if causal else None))
    plain = torch.where(torch.isnan(plain), torch.zeros_like(plain), plain)
    assert _cos(out.cpu(), plain) > 0.99
    # the torch op is the same path, with an explicit softmax scale
    out2 = torch.ops.tensorrt.b200_fp8_sdpa(q.cuda(), k.cuda(), v.cuda(), aq.cuda(), ak.cuda(), av.cuda(), causal, 1.0 / D ** 0.5)
    assert torch.equal(out2, out)


@pytest.mark.gpu
def test_fp8_sdpa_codes_of_the_transposed_value_operand(b200):
    """b200q_fp8_quantize_transpose: the codes of V, transposed per head with zero padding, are the
    oracle's codes bit for bit."""
    from tensorrt_b200 import _lib

    lib = _lib.load()
    g = torch.Generator().manual_seed(2)
    heads, S, D = 3, 77, 48
    v = (torch.randn(heads, S, D, generator=g) * 3).bfloat16()
    amax = v.float().abs().max()
    codes, scale = o.fp8_quantize(v, amax)
    stride = 80
    out = torch.full((heads, D, stride), 0xAA, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(1, device="cuda")
    vd, ad = v.cuda(), amax.reshape(1).cuda()
    assert lib.b200q_fp8_quantize_transpose(vd.data_ptr(), 2, heads, S, D, ad.data_ptr(), out.data_ptr(), stride, sc.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert sc.item() == scale.item()
    assert torch.equal(out[:, :, :S].cpu(), codes.transpose(1, 2)) and int(out[:, :, S:].max()) == 0


def test_fx_pass_rewrites_the_fp8_mha_pattern(b200):
    """quantize_op on Q, K, V in front of scaled_dot_product_attention becomes one b200_fp8_sdpa node; an
    attention with an explicit mask, or with one input not quantized, is left alone."""
    from tensorrt_b200.fx_passes import fuse_fp8_sdpa

    class Mha(torch.nn.Module):
        def __init__(self, mask=False, quantize_v=True, causal=True):
            super().__init__()
            for n in ("amax_q", "amax_k", "amax_v"):
                self.register_buffer(n, torch.tensor(6.0))
            self.register_buffer("m", torch.ones(33, 33, dtype=torch.bool))
            self.mask, self.quantize_v, self.causal = mask, quantize_v, causal

        def forward(self, q, k, v):
            qo = torch.ops.tensorrt.quantize_op
            q8, k8 = qo(q, self.amax_q, 8, 4, False, False), qo(k, self.amax_k, 8, 4, False, False)
            v8 = qo(v, self.amax_v, 8, 4, False, False) if self.quantize_v else v
            if self.mask:
                return torch.nn.functional.scaled_dot_product_attention(q8, k8, v8, attn_mask=self.m)
            return torch.nn.functional.scaled_dot_product_attention(q8, k8, v8, is_causal=self.causal)

    gm = torch.fx.symbolic_trace(Mha())
    assert fuse_fp8_sdpa(gm) == 1
    names = [str(n.target) for n in gm.graph.nodes if n.op == "call_function"]
    assert sum("b200_fp8_sdpa" in t for t in names) == 1 and not any("quantize_op" in t or "scaled_dot" in t for t in names)
    node = next(n for n in gm.graph.nodes if "b200_fp8_sdpa" in str(n.target))
    assert node.args[6] is True and node.args[7] == -1.0
    y = gm.to("meta")(*(torch.empty(2, 4, 33, 64, dtype=torch.float16, device="meta") for _ in range(3)))
    assert y.shape == (2, 4, 33, 64) and y.dtype == torch.float16
    assert fuse_fp8_sdpa(gm) == 0
    for kw in ({"mask": True}, {"quantize_v": False}):
        g2 = torch.fx.symbolic_trace(Mha(**kw))
        assert fuse_fp8_sdpa(g2) == 0


@pytest.mark.gpu
def test_rewritten_mha_graph_matches_eager_quantized_attention(b200):
    """The reference's test model (quantize_op on Q, K, V feeding SDPA), rewritten and run on the device,
    against the same module run eagerly (fake-quant ops + torch attention) and against plain attention."""
    from tensorrt_b200.fx_passes import fuse_fp8_sdpa

    class Mha(torch.nn.Module):
        def __init__(self):
            super().__init__()
            for n in ("amax_q", "amax_k", "amax_v"):
                self.register_buffer(n, torch.tensor(6.0))

        def forward(self, q, k, v):
            qo = torch.ops.tensorrt.quantize_op
            return torch.nn.functional.scaled_dot_product_attention(qo(q, self.amax_q, 8, 4, False, False), qo(k, self.amax_k, 8, 4, False, False),
                                                                    qo(v, self.amax_v, 8, 4, False, False))

    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 2, 32, 64, dtype=torch.float16).cuda() for _ in range(3))
    m = Mha().cuda()
    eager = m(q, k, v)
    gm = torch.fx.symbolic_trace(m)
    assert fuse_fp8_sdpa(gm) == 1
    out = gm(q, k, v)
    plain = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    assert _cos(out, plain) > 0.99 and _cos(out, eager) > 0.995
