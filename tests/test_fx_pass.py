"""FX rewrite of Q/DQ-wrapped linears (tensorrt_b200/fx_passes.py): graph structure and shape
propagation on CPU (meta tensors), numerics against the unfused graph on the GPU."""
import pytest
import torch

import oracle as o


class QdqLinear(torch.nn.Module):
    """linear(input_quantizer(x), weight_quantizer(W), b) as the reference's calibrated modules
    call it (FP8: quantize_op; NVFP4: dynamic_block_quantize_op)."""

    def __init__(self, n, k, mode="fp8", bias=True, seed=0, dtype=torch.bfloat16):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.mode = mode
        self.weight = torch.nn.Parameter((torch.randn(n, k, generator=g) * 0.02).to(dtype))
        self.bias = torch.nn.Parameter((torch.randn(n, generator=g) * 0.01).to(dtype)) if bias else None
        self.register_buffer("x_amax", torch.tensor(4.0))
        self.register_buffer("w_amax", self.weight.detach().float().abs().max())

    def q(self, t, amax):
        if self.mode == "fp8":
            return torch.ops.tensorrt.quantize_op(t, amax, 8, 4, False, False)
        return torch.ops.tensorrt.dynamic_block_quantize_op(t, 16, amax, 4, 2, 8, 4)

    def forward(self, x):
        return torch.nn.functional.linear(self.q(x, self.x_amax), self.q(self.weight, self.w_amax), self.bias)


class TwoLayer(torch.nn.Module):
    def __init__(self, mode):
        super().__init__()
        self.a, self.b = QdqLinear(64, 32, mode, seed=1), QdqLinear(48, 64, mode, bias=False, seed=2)

    def forward(self, x):
        return self.b(torch.nn.functional.silu(self.a(x)))


def _targets(gm):
    return [str(n.target) for n in gm.graph.nodes if n.op == "call_function"]


@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
@pytest.mark.parametrize("how", ["trace", "export"])
def test_rewrite_structure_and_meta_shapes(b200, mode, how):
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    m = TwoLayer(mode)
    if how == "trace":
        gm = torch.fx.symbolic_trace(m)
    else:
        gm = torch.export.export(m, (torch.randn(4, 32).bfloat16(),)).module()
    assert fuse_quantized_linear(gm) == 2
    names = _targets(gm)
    assert not any("linear" in t or "tensorrt.quantize_op" in t or "dynamic_block_quantize_op" in t for t in names), names
    kind = "fp8" if mode == "fp8" else "nvfp4"
    assert sum(f"b200_{kind}_gemm" in t for t in names) == 2
    assert sum(f"b200_{kind}_quantize" in t for t in names) == 4      # CPU weights are not folded
    assert fuse_quantized_linear(gm) == 0                              # idempotent
    if how == "trace":
        y = gm.to("meta")(torch.empty(3, 5, 32, dtype=torch.bfloat16, device="meta"))
        assert y.shape == (3, 5, 48) and y.dtype == torch.bfloat16


def test_rewrite_leaves_other_graphs_alone(b200):
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    class OnlyInput(torch.nn.Module):          # weight not quantized: not the Q/DQ-linear pattern
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.randn(16, 32).bfloat16())
            self.register_buffer("a", torch.tensor(1.0))

        def forward(self, x):
            return torch.nn.functional.linear(torch.ops.tensorrt.quantize_op(x, self.a, 8, 4, False, False), self.w)

    class Mixed(torch.nn.Module):              # FP8 input with an NVFP4 weight: no single GEMM kind
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.randn(16, 32).bfloat16())
            self.register_buffer("a", torch.tensor(1.0))

        def forward(self, x):
            xq = torch.ops.tensorrt.quantize_op(x, self.a, 8, 4, False, False)
            wq = torch.ops.tensorrt.dynamic_block_quantize_op(self.w, 16, self.a, 4, 2, 8, 4)
            return torch.nn.functional.linear(xq, wq)

    class Int8(torch.nn.Module):               # (8, 0) is INT8 in the reference, not E4M3
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.randn(16, 32).bfloat16())
            self.register_buffer("a", torch.tensor(1.0))

        def forward(self, x):
            xq = torch.ops.tensorrt.quantize_op(x, self.a, 8, 0, False, False)
            wq = torch.ops.tensorrt.quantize_op(self.w, self.a, 8, 0, False, False)
            return torch.nn.functional.linear(xq, wq)

    for cls in (OnlyInput, Mixed, Int8):
        gm = torch.fx.symbolic_trace(cls())
        before = _targets(gm)
        assert fuse_quantized_linear(gm) == 0
        assert _targets(gm) == before


def test_shared_quantize_node_is_kept_for_its_other_user(b200):
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    class Shared(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = QdqLinear(16, 32)

        def forward(self, x):
            xq = self.lin.q(x, self.lin.x_amax)
            y = torch.nn.functional.linear(xq, self.lin.q(self.lin.weight, self.lin.w_amax), self.lin.bias)
            return y, xq.sum()

    gm = torch.fx.symbolic_trace(Shared())
    assert fuse_quantized_linear(gm) == 1
    names = _targets(gm)
    assert sum("tensorrt.quantize_op" in t for t in names) == 1       # still feeds xq.sum()
    assert sum("b200_fp8_gemm" in t for t in names) == 1


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
def test_rewritten_graph_matches_unfused_graph_on_gpu(b200, mode):
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    torch.manual_seed(11)
    m = QdqLinear(512, 256, mode, seed=3).cuda()
    x = torch.randn(6, 40, 256, device="cuda").bfloat16()
    m.x_amax.copy_(x.float().abs().max())
    ref = m(x)
    gm = torch.fx.symbolic_trace(m)
    assert fuse_quantized_linear(gm) == 1
    names = _targets(gm)
    kind = "fp8" if mode == "fp8" else "nvfp4"
    assert sum(f"b200_{kind}_quantize" in t for t in names) == 1      # the weight was folded into buffers
    assert any(n.startswith("_b200q_w0_") for n, _ in gm.named_buffers())
    y = gm(x)
    assert y.shape == ref.shape and y.dtype == ref.dtype
    assert o.rel_l2(y.float().cpu(), ref.float().cpu()) <= 1e-2
    # fp16 input: the rewritten graph returns the linear's dtype
    m16 = QdqLinear(128, 64, mode, seed=4, dtype=torch.float16).cuda()
    x16 = torch.randn(32, 64, device="cuda").half()
    ep = torch.export.export(m16, (x16,))
    g16 = ep.module()
    assert fuse_quantized_linear(g16) == 1
    y16 = g16(x16)
    assert y16.dtype == torch.float16
    assert o.rel_l2(y16.float().cpu(), m16(x16).float().cpu()) <= 1e-2


@pytest.mark.parametrize("form", ["mm", "matmul", "addmm", "method_t"])
def test_matmul_and_addmm_forms_are_the_same_linear(b200, form):
    """`aten.linear` reaches the converters as mm / addmm with a transposed weight in distributed
    mode (lowering/_decompositions.py:738-745); those forms are rewritten too."""
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = QdqLinear(48, 32)

        def forward(self, x):
            xq = self.lin.q(x, self.lin.x_amax)
            wq = self.lin.q(self.lin.weight, self.lin.w_amax)
            if form == "mm":
                return torch.ops.aten.mm.default(xq, torch.ops.aten.t.default(wq))
            if form == "matmul":
                return torch.matmul(xq, torch.ops.aten.permute.default(wq, [1, 0]))
            if form == "addmm":
                return torch.ops.aten.addmm.default(self.lin.bias, xq, torch.ops.aten.transpose.int(wq, 0, 1))
            return torch.mm(xq, wq.t())

    gm = torch.fx.symbolic_trace(M())
    assert fuse_quantized_linear(gm) == 1
    names = _targets(gm)
    assert sum("b200_fp8_gemm" in t for t in names) == 1
    assert not any("quantize_op" in t or "aten.mm" in t or "addmm" in t or "matmul" in t or "aten.t." in t or "permute" in t
                   or "transpose" in t for t in names), names
    gemm = next(n for n in gm.graph.nodes if "b200_fp8_gemm" in str(n.target))
    assert ("gemm_bias" in str(gemm.target)) == (form == "addmm")    # addmm's first argument is the bias
    assert len(gemm.args) == (5 if form == "addmm" else 4)
    y = gm.to("meta")(torch.empty(7, 32, dtype=torch.bfloat16, device="meta"))
    assert y.shape == (7, 48)
    # a plain matmul of two quantized activations (no transposed weight) is not a linear
    class Plain(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("a", torch.tensor(1.0))

        def forward(self, x, y):
            q = lambda t: torch.ops.tensorrt.quantize_op(t, self.a, 8, 4, False, False)  # noqa: E731
            return torch.matmul(q(x), q(y))

    gm2 = torch.fx.symbolic_trace(Plain())
    assert fuse_quantized_linear(gm2) == 0


def test_linears_sharing_one_input_quantizer_share_one_quantize_node(b200):
    """q/k/v (or gate/up) projections read the same quantized activation: the rewrite inserts ONE
    real-quant node for it, not one per linear."""
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    class Qkv(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.v = QdqLinear(64, 32, seed=1), QdqLinear(16, 32, seed=2), QdqLinear(16, 32, seed=3)

        def forward(self, x):
            xq = self.q.q(x, self.q.x_amax)
            outs = [torch.nn.functional.linear(xq, m.q(m.weight, m.w_amax), m.bias) for m in (self.q, self.k, self.v)]
            return torch.cat(outs, dim=-1)

    gm = torch.fx.symbolic_trace(Qkv())
    assert fuse_quantized_linear(gm) == 3
    names = _targets(gm)
    assert sum("b200_fp8_gemm_bias" in t for t in names) == 3
    assert sum("b200_fp8_quantize" in t for t in names) == 1 + 3          # one activation quantize + 3 unfolded CPU weights
    assert not any("tensorrt.quantize_op" in t for t in names)
    y = gm.to("meta")(torch.empty(5, 32, dtype=torch.bfloat16, device="meta"))
    assert y.shape == (5, 96)


def test_keyword_arguments_and_unsigned_quantizers(b200):
    """The quantize ops are matched by schema, so keyword forms fuse like positional ones; an
    unsigned or narrow-range quantizer is a different arithmetic and is left alone."""
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    def build(**flags):
        class M(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.w = torch.nn.Parameter(torch.randn(16, 32).bfloat16())
                self.register_buffer("a", torch.tensor(1.0))

            def forward(self, x):
                q = torch.ops.tensorrt.quantize_op
                xq = q(x, self.a, num_bits=8, exponent_bits=4, unsigned=flags.get("unsigned", False),
                       narrow_range=flags.get("narrow_range", False))
                wq = q(self.w, amax=self.a, num_bits=8, exponent_bits=4, unsigned=False, narrow_range=False)
                return torch.nn.functional.linear(xq, wq)
        return torch.fx.symbolic_trace(M())

    assert fuse_quantized_linear(build()) == 1
    for flags in ({"unsigned": True}, {"narrow_range": True}):
        gm = build(**flags)
        before = _targets(gm)
        assert fuse_quantized_linear(gm) == 0 and _targets(gm) == before


def test_addmm_with_alpha_and_beta(b200):
    """addmm = beta * input + alpha * (x @ W^T) (conversion/impl/addmm.py:12-34): with factors other
    than 1 the bias cannot ride in the GEMM epilogue; the scaling stays as nodes behind the GEMM."""
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = QdqLinear(48, 32)

        def forward(self, x):
            xq = self.lin.q(x, self.lin.x_amax)
            wq = self.lin.q(self.lin.weight, self.lin.w_amax)
            return torch.ops.aten.addmm.default(self.lin.bias, xq, torch.ops.aten.t.default(wq), beta=0.5, alpha=2.0)

    gm = torch.fx.symbolic_trace(M())
    assert fuse_quantized_linear(gm) == 1
    names = _targets(gm)
    assert sum("b200_fp8_gemm" in t for t in names) == 1 and not any("gemm_bias" in t or "addmm" in t for t in names)
    assert any("aten.mul" in t for t in names) and any("aten.add" in t for t in names)
    add = next(n for n in gm.graph.nodes if "aten.add" in str(n.target))
    assert add.kwargs == {"alpha": 0.5}
    mul = next(n for n in gm.graph.nodes if "aten.mul" in str(n.target))
    assert mul.args[1] == 2.0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
@pytest.mark.parametrize("form", ["mm", "matmul3d", "addmm", "addmm_ab"])
def test_mm_matmul_addmm_forms_match_the_unfused_graph_on_gpu(b200, mode, form):
    """The forms `aten.linear` decomposes to in distributed mode (lowering/_decompositions.py:738-745),
    rewritten and run on the device, against the same graph left unfused (fake-quant ops + bf16
    matmul).  Tolerance: rel-L2 <= 1e-2, the bar of the linear form."""
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = QdqLinear(384, 256, mode, seed=5)

        def forward(self, x):
            xq = self.lin.q(x, self.lin.x_amax)
            wq = self.lin.q(self.lin.weight, self.lin.w_amax)
            if form == "mm":
                return torch.ops.aten.mm.default(xq, torch.ops.aten.t.default(wq))
            if form == "matmul3d":
                return torch.matmul(xq, torch.ops.aten.permute.default(wq, [1, 0]))
            if form == "addmm":
                return torch.ops.aten.addmm.default(self.lin.bias, xq, torch.ops.aten.transpose.int(wq, 0, 1))
            return torch.ops.aten.addmm.default(self.lin.bias, xq, torch.ops.aten.t.default(wq), beta=0.5, alpha=2.0)

    m = M().cuda()
    g = torch.Generator().manual_seed(17)
    shape = (4, 50, 256) if form == "matmul3d" else (200, 256)
    x = torch.randn(*shape, generator=g).bfloat16().cuda()
    m.lin.x_amax.copy_(x.float().abs().max())
    ref = m(x)
    gm = torch.fx.symbolic_trace(m)
    assert fuse_quantized_linear(gm) == 1
    assert not hasattr(gm.lin, "weight")                # the folded bf16 weight is gone, only its codes remain
    y = gm(x)
    torch.cuda.synchronize()
    assert b200.capi.device_status() == 0
    assert y.shape == ref.shape and y.dtype == ref.dtype
    assert o.rel_l2(y.float().cpu(), ref.float().cpu()) <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_plugin_form_is_one_node_per_linear_and_matches_on_gpu(b200, mode, dtype):
    """plugin_form=True: each linear with a constant weight is ONE `b200_*_linear[_bias]` node with
    tensor-only arguments, activation first, result in the activation's dtype (what the reference's
    plugin generator can describe); numerics as the two-node form."""
    from tensorrt_b200.fx_passes import fuse_quantized_linear

    m = TwoLayer(mode).to(dtype).cuda()
    x = torch.randn(3, 40, 32, device="cuda").to(dtype)
    m.a.x_amax.copy_(x.float().abs().max())
    m.b.x_amax.copy_(torch.nn.functional.silu(m.a(x)).float().abs().max())
    ref = m(x)
    gm = torch.fx.symbolic_trace(m)
    assert fuse_quantized_linear(gm, plugin_form=True) == 2
    names = _targets(gm)
    kind = "fp8" if mode == "fp8" else "nvfp4"
    assert sum(f"b200_{kind}_linear_bias" in t for t in names) == 1 and sum(f"b200_{kind}_linear" in t for t in names) == 2
    assert not any("quantize" in t or "gemm" in t for t in names), names
    for n in gm.graph.nodes:
        if "b200_" in str(n.target):
            assert all(isinstance(a, torch.fx.Node) for a in n.args)
    y = gm(x)
    assert y.dtype == dtype and y.shape == ref.shape
    # two quantized layers back to back against the fake-quant graph: the second layer sees slightly
    # different inputs on the two sides, NVFP4's coarse grid amplifies that more than FP8's
    assert o.rel_l2(y.float().cpu().detach(), ref.float().cpu().detach()) <= (2e-2 if mode == "fp8" else 5e-2)


def _all_reduce_graph(extra_user: bool):
    """x -> all_reduce -> wait_tensor -> relu, built node by node (functional collectives as they
    appear in an exported tensor-parallel graph)."""
    c10d = torch.ops._c10d_functional
    g = torch.fx.Graph()
    x = g.placeholder("x")
    ar = g.call_function(c10d.all_reduce.default, (x, "sum", "0"))
    w = g.call_function(c10d.wait_tensor.default, (ar,))
    out = g.call_function(torch.relu, (w,))
    if extra_user:
        out = g.call_function(torch.add, (out, ar))
    g.output(out)
    return torch.fx.GraphModule(torch.nn.Module(), g)


def test_all_reduce_plus_wait_becomes_the_fused_op(b200):
    from tensorrt_b200.fx_passes import fuse_all_reduce_wait

    gm = _all_reduce_graph(extra_user=False)
    assert fuse_all_reduce_wait(gm) == 1
    names = _targets(gm)
    assert sum("tensorrt.fused_nccl_all_reduce" in t for t in names) == 1
    assert not any("_c10d_functional" in t for t in names), names
    node = next(n for n in gm.graph.nodes if "fused_nccl_all_reduce" in str(n.target))
    assert node.args[1:] == ("sum", "0")                               # exactly (inp, reduce_op, group_name)
    assert fuse_all_reduce_wait(gm) == 0
    # without a process group the eager op is the identity (single rank), out of place
    x = torch.randn(4, 8)
    gm.graph.lint()
    node.args = (node.args[0], "sum", "default")
    gm.recompile()
    assert torch.equal(gm(x), torch.relu(x))
    # an all-reduce that something else also reads keeps its wait
    gm2 = _all_reduce_graph(extra_user=True)
    before = _targets(gm2)
    assert fuse_all_reduce_wait(gm2) == 0 and _targets(gm2) == before


class GatedMlp(torch.nn.Module):
    """down(silu(gate(x)) * up(x)) with Q/DQ on every linear input and weight, gate and up sharing the
    input quantizer (per-tensor amax, as after calibration)."""

    def __init__(self, hidden=256, ffn=384, bias=False):
        super().__init__()
        self.gate, self.up = QdqLinear(ffn, hidden, bias=bias, seed=11), QdqLinear(ffn, hidden, bias=bias, seed=12)
        self.down = QdqLinear(hidden, ffn, bias=False, seed=13)

    def forward(self, x):
        xq = self.gate.q(x, self.gate.x_amax)
        g = torch.nn.functional.linear(xq, self.gate.q(self.gate.weight, self.gate.w_amax), self.gate.bias)
        u = torch.nn.functional.linear(xq, self.up.q(self.up.weight, self.up.w_amax), self.up.bias)
        return self.down(torch.nn.functional.silu(g) * u)


def test_gated_mlp_pass_leaves_unfolded_or_biased_linears_alone(b200):
    """On CPU the weights are not folded into constants, so there is nothing the pass may stack."""
    from tensorrt_b200.fx_passes import fuse_gated_mlp, fuse_quantized_linear

    gm = torch.fx.symbolic_trace(GatedMlp())
    assert fuse_quantized_linear(gm) == 3
    assert fuse_gated_mlp(gm) == 0
    assert sum("b200_fp8_gemm" in t for t in _targets(gm)) == 3


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [8, 300])
def test_gated_mlp_becomes_one_gemm_with_the_activation_in_its_epilogue(b200, tokens):
    """gate and up linears + silu * up -> one b200_fp8_gemm_silu_mul node on the stacked weight (fewer than 256
    tokens run GEMM + activation kernel inside the op, more run the fused epilogue).  Against the graph before
    the pass, where torch's own silu and mul round to bf16 twice, the result differs by that rounding only; a
    bias or an F that is not a multiple of 128 is left alone."""
    from tensorrt_b200.fx_passes import fuse_gated_mlp, fuse_quantized_linear

    x = (torch.randn(tokens, 256, generator=torch.Generator().manual_seed(3)) * 1.5).bfloat16().cuda()
    gm = torch.fx.symbolic_trace(GatedMlp().cuda())
    assert fuse_quantized_linear(gm) == 3
    before = gm(x)
    assert fuse_gated_mlp(gm) == 1
    names = _targets(gm)
    # the activation's static quantizer went into the epilogue too: the node returns (codes, scale)
    assert sum("b200_fp8_gemm_silu_mul_quant" in t for t in names) == 1 and not any("silu." in t or t.endswith("silu") for t in names if "gemm" not in t)
    assert sum("b200_fp8_gemm" in t for t in names) == 2               # the fused node and the down projection
    assert sum("b200_fp8_quantize" in t for t in names) == 1           # x only: all weights folded, the activation quantized in the GEMM
    after = gm(x)
    assert o.rel_l2(after.float().cpu(), before.float().cpu()) < 2e-2   # through the FP8 re-quantization in front of the down projection
    assert fuse_gated_mlp(gm) == 0                                      # idempotent
    leftovers = [n for n, _ in gm.named_buffers() if n.startswith("_b200q_w")]
    assert len(leftovers) == 2, leftovers                               # codes and scales of the down projection only
    for model in (GatedMlp(bias=True), GatedMlp(ffn=320)):
        gm2 = torch.fx.symbolic_trace(model.cuda())
        assert fuse_quantized_linear(gm2) == 3
        assert fuse_gated_mlp(gm2) == 0
