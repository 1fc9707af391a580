"""FX rewrite: Q/DQ-wrapped linears -> real-quant GEMM nodes.

The reference keeps `linear(input_quantizer(x), weight_quantizer(W), bias)` as three nodes
(`tensorrt::quantize_op` / `tensorrt::dynamic_block_quantize_op` twice, then `aten.linear`;
converters at py/torch_tensorrt/dynamo/conversion/aten_ops_converters.py:904-960 and :4197-4213)
and relies on TensorRT to fuse the Q/DQ pairs into an FP8/FP4 GEMM.  `fuse_quantized_linear`
does that fusion on the graph itself:

    xq = quantize_op(x, ax, 8, 4, False, False)
    wq = quantize_op(W, aw, 8, 4, False, False)          ==>   xc, xs = b200_fp8_quantize(x, ax)
    y  = linear(xq, wq, b)                                     wc, ws = b200_fp8_quantize(W, aw)
                                                               y = b200_fp8_gemm(xc, xs, wc, ws, b)

(`mm(xq, wq.t())`, `matmul(xq, wq.t())` and `addmm(b, xq, wq.t(), beta=, alpha=)` are recognised as the
same linear: they are what `aten.linear` decomposes to in the reference's distributed mode,
py/torch_tensorrt/dynamo/lowering/_decompositions.py:738-745; with `alpha`/`beta` other than 1 the
scaling of py/torch_tensorrt/dynamo/conversion/impl/addmm.py:12-34 is kept as separate nodes after
the GEMM.)  Linears that share one activation quantizer (q/k/v, gate/up) share one inserted
quantize node.  With `plugin_form=True` and a constant weight each linear becomes ONE node,
`b200_fp8_linear[_bias](x, ax, wc, ws[, b])`, whose arguments are all tensors with the activation
first and whose result has the activation's dtype: the form
`torch_tensorrt.dynamo.conversion.plugins.custom_op` can turn into a TensorRT plugin.

and the same with `dynamic_block_quantize_op(.., 16, amax, 4, 2, 8, 4)` -> `b200_nvfp4_*`.
The fake-quantized bf16 tensors are never materialised; the result differs from the unfused
graph only by the GEMM's accumulation (fp32 over code products instead of bf16 operands).
A weight that is a constant of the graph module on a CUDA device is quantized once at rewrite
time and replaced by its codes and scales (`fold_weights=True`).

The rewritten nodes are `torch.ops.tensorrt.b200_*` dispatcher ops with Meta kernels, so the
graph still traces under FakeTensorMode and each node can be handed to
`torch_tensorrt.dynamo.conversion.plugins.custom_op` (see plugin.register_with_torch_tensorrt).
"""
from __future__ import annotations

import operator

import torch
from torch import fx

_FP8_ARGS = (8, 4)          # num_bits, exponent_bits of quantize_op for E4M3
_NVFP4_ARGS = (16, 4, 2, 8, 4)  # block_size, num_bits, exponent_bits, scale_num_bits, scale_exponent_bits


def _is_op(node: fx.Node, packet) -> bool:
    if node.op != "call_function":
        return False
    t = node.target
    return t is packet or t is getattr(packet, "default", None)


def _linear_targets():
    return (torch.nn.functional.linear, torch.ops.aten.linear, torch.ops.aten.linear.default)


def _transposed(node):
    """W behind `W.t()` / `W.T`-style nodes (aten.t, transpose(0, 1), permute([1, 0])), else None."""
    if not isinstance(node, fx.Node):
        return None
    if node.op == "call_function":
        a = torch.ops.aten
        if node.target in (a.t, a.t.default):
            return node.args[0]
        if node.target in (a.transpose, a.transpose.int, torch.transpose) and tuple(node.args[1:3]) in ((0, 1), (1, 0), (-1, -2), (-2, -1)):
            return node.args[0]
        if node.target in (a.permute, a.permute.default, torch.permute) and list(node.args[1]) == [1, 0]:
            return node.args[0]
    if node.op == "call_method" and node.target == "t":
        return node.args[0]
    return None


def _as_linear(node: fx.Node):
    """(input, weight, bias, alpha, beta) when `node` computes alpha * (input @ weight^T) + beta * bias in
    one of the forms the reference converts (aten_ops_converters.py:4197-4213 linear, :779-799 matmul,
    :3477-3500 addmm, the form `aten.linear` decomposes to in distributed mode), else None."""
    if node.op != "call_function":
        return None
    a = torch.ops.aten
    if node.target in _linear_targets() and len(node.args) >= 2:
        return node.args[0], node.args[1], (node.args[2] if len(node.args) > 2 else node.kwargs.get("bias")), 1, 1
    if node.target in (a.mm, a.mm.default, a.matmul, a.matmul.default, torch.matmul, torch.mm) and len(node.args) == 2:
        w = _transposed(node.args[1])
        return (node.args[0], w, None, 1, 1) if w is not None else None
    if node.target in (a.addmm, a.addmm.default, torch.addmm) and len(node.args) == 3:
        if set(node.kwargs) - {"alpha", "beta"}:
            return None
        alpha, beta = node.kwargs.get("alpha", 1), node.kwargs.get("beta", 1)
        if not isinstance(alpha, (int, float)) or not isinstance(beta, (int, float)):
            return None
        w = _transposed(node.args[2])
        return (node.args[1], w, node.args[0], alpha, beta) if w is not None else None
    return None


def _bound_args(node: fx.Node, packet):
    """Arguments of an op node by schema name (positional and keyword forms alike), or None."""
    schema = packet.default._schema
    names = [a.name for a in schema.arguments]
    if len(node.args) > len(names) or set(node.kwargs) - set(names):
        return None
    bound = dict(zip(names, node.args))
    for k, v in node.kwargs.items():
        if k in bound:
            return None
        bound[k] = v
    for a in schema.arguments:
        if a.name not in bound:
            if not a.has_default_value():
                return None
            bound[a.name] = a.default_value
    return [bound[n] for n in names]


def _match_fp8(node: fx.Node):
    """quantize_op(input, amax, 8, 4, unsigned=False, narrow_range=False) -> (input, amax).  The
    signed, full-range E4M3 case only: anything else is left to the unfused graph."""
    if not _is_op(node, torch.ops.tensorrt.quantize_op):
        return None
    args = _bound_args(node, torch.ops.tensorrt.quantize_op)
    if args is None or tuple(args[2:4]) != _FP8_ARGS or args[4] is not False or args[5] is not False:
        return None
    return args[0], args[1]


def _match_nvfp4(node: fx.Node):
    """dynamic_block_quantize_op(input, 16, amax, 4, 2, 8, 4) -> (input, amax)."""
    if not _is_op(node, torch.ops.tensorrt.dynamic_block_quantize_op):
        return None
    args = _bound_args(node, torch.ops.tensorrt.dynamic_block_quantize_op)
    if args is None or (args[1],) + tuple(args[3:7]) != _NVFP4_ARGS:
        return None
    return args[0], args[2]


def _const_tensor(gm: fx.GraphModule, node):
    """Tensor behind a get_attr node, else None."""
    if not isinstance(node, fx.Node) or node.op != "get_attr":
        return None
    obj = gm
    for part in node.target.split("."):
        obj = getattr(obj, part, None)
        if obj is None:
            return None
    return obj if isinstance(obj, torch.Tensor) else None


def _out_dtype(node: fx.Node):
    val = node.meta.get("val")
    if isinstance(val, torch.Tensor):
        return val.dtype
    tm = node.meta.get("tensor_meta")
    return getattr(tm, "dtype", None)


def _drop_unused_constant(gm: fx.GraphModule, node) -> None:
    """Delete the module attribute behind a get_attr node that nothing in the graph reads any more
    (the bf16 weight of a linear whose codes were folded in: keeping it would double weight memory)."""
    if not isinstance(node, fx.Node) or node.op != "get_attr" or node.users:
        return
    target = node.target
    gm.graph.erase_node(node)
    if any(n.op == "get_attr" and n.target == target for n in gm.graph.nodes):
        return
    *path, leaf = target.split(".")
    owner = gm
    for part in path:
        owner = getattr(owner, part, None)
        if owner is None:
            return
    if hasattr(owner, leaf):
        delattr(owner, leaf)


def fuse_quantized_linear(gm: fx.GraphModule, fold_weights: bool = True, plugin_form: bool = False) -> int:
    """Rewrite every linear whose input and weight both come from matching FP8 (or both from
    NVFP4) quantize ops.  Returns the number of linears rewritten; the module is recompiled
    in place.  Quantize nodes left without users are removed; a quantize node that still feeds
    something else is kept for that user.  Constant weights (`fold_weights`) are quantized once,
    here, and their bf16 originals are deleted from the module when nothing else reads them.
    `plugin_form`: emit one `b200_*_linear[_bias]` node per linear with a folded weight (see the
    module docstring); linears whose weight is not a constant keep the quantize + GEMM form."""
    from . import ops

    ops.load_ops()
    t = torch.ops.tensorrt
    graph, n_fused = gm.graph, 0
    n_const = sum(1 for name, _ in gm.named_buffers(recurse=False) if name.startswith("_b200q_w") and name.endswith("_0"))
    act_cache: dict = {}       # (mode, input node, amax node) -> getitem nodes of the one inserted quantize
    for node in list(graph.nodes):
        form = _as_linear(node)
        if form is None:
            continue
        xq, wq, bias, alpha, beta = form
        if not isinstance(xq, fx.Node) or not isinstance(wq, fx.Node):
            continue
        mode, mx, mw = "fp8", _match_fp8(xq), _match_fp8(wq)
        if mx is None or mw is None:
            mode, mx, mw = "nvfp4", _match_nvfp4(xq), _match_nvfp4(wq)
        if mx is None or mw is None:
            continue
        quant = t.b200_fp8_quantize.default if mode == "fp8" else t.b200_nvfp4_quantize.default
        parts = 2 if mode == "fp8" else 3
        epilogue_bias = bias if (bias is not None and alpha == 1 and beta == 1) else None
        w_src = mw[0]
        with graph.inserting_before(node):
            w_const, a_const = _const_tensor(gm, mw[0]), _const_tensor(gm, mw[1])
            folded = fold_weights and w_const is not None and a_const is not None and w_const.is_cuda
            if folded:
                with torch.no_grad():
                    tensors = quant(w_const.detach(), a_const.detach().to(w_const.device))
                w_parts = []
                for i, tensor in enumerate(tensors):
                    name = f"_b200q_w{n_const}_{i}"
                    gm.register_buffer(name, tensor)
                    w_parts.append(graph.get_attr(name))
                n_const += 1
            else:
                ws = graph.call_function(quant, (mw[0], mw[1]))
                w_parts = [graph.call_function(operator.getitem, (ws, i)) for i in range(parts)]
            if plugin_form and folded:
                name = f"b200_{mode}_linear" + ("_bias" if epilogue_bias is not None else "")
                args = (mx[0], mx[1], *w_parts) + ((epilogue_bias,) if epilogue_bias is not None else ())
                out = graph.call_function(getattr(t, name).default, args)       # result in the activation's dtype
            else:
                key = (mode, mx[0], mx[1])
                x_parts = act_cache.get(key)
                if x_parts is None:
                    # placed right after its inputs so that every later linear sharing it can use it
                    anchor = max((n for n in mx if isinstance(n, fx.Node)), key=lambda n: _node_index(graph, n))
                    with graph.inserting_after(anchor):
                        xs = graph.call_function(quant, (mx[0], mx[1]))
                    with graph.inserting_after(xs):
                        x_parts = [graph.call_function(operator.getitem, (xs, i)) for i in reversed(range(parts))][::-1]
                    act_cache[key] = x_parts
                name = f"b200_{mode}_gemm" + ("_bias" if epilogue_bias is not None else "")
                args = (*x_parts, *w_parts) + ((epilogue_bias,) if epilogue_bias is not None else ())
                out = graph.call_function(getattr(t, name).default, args)
                dtype = _out_dtype(node)
                if dtype is not None and dtype != torch.bfloat16:
                    out = graph.call_method("to", (out, dtype))
            if epilogue_bias is None and bias is not None:
                # addmm with alpha / beta != 1 (impl/addmm.py:12-34): beta * input + alpha * (x @ W^T)
                if alpha != 1:
                    out = graph.call_function(torch.ops.aten.mul.Tensor, (out, alpha))
                out = graph.call_function(torch.ops.aten.add.Tensor, (out, bias), {"alpha": beta})
        out.meta.update({k: v for k, v in node.meta.items() if k in ("val", "tensor_meta")})
        node.replace_all_uses_with(out)
        dangling = [a for a in node.all_input_nodes if _transposed(a) is wq]
        graph.erase_node(node)
        for tnode in dangling:
            if not tnode.users:
                graph.erase_node(tnode)
        for q in (xq, wq):
            if not q.users:
                graph.erase_node(q)
        if folded:
            _drop_unused_constant(gm, w_src)
        n_fused += 1
    if n_fused:
        graph.eliminate_dead_code()
        graph.lint()
        gm.recompile()
    return n_fused


def _node_index(graph: fx.Graph, node: fx.Node) -> int:
    for i, n in enumerate(graph.nodes):
        if n is node:
            return i
    return -1


def fuse_fp8_sdpa(gm: fx.GraphModule) -> int:
    """`scaled_dot_product_attention(quantize_op(q), quantize_op(k), quantize_op(v), ..)` with all three
    quantizers FP8 E4M3 becomes one `tensorrt::b200_fp8_sdpa` node: the pattern the reference detects in
    py/torch_tensorrt/dynamo/lowering/passes/annotate_fp8_sdpa.py:34-76 (it marks the node with the softmax
    quantization scale 1/448 and lets TensorRT fuse an FP8 attention kernel; here the kernel is the node).
    Left alone: an explicit attn_mask, dropout, quantizers with a per-row amax the graph can prove
    (constant amax with more than one element).  Returns the number of nodes rewritten."""
    from . import ops

    ops.load_ops()
    a = torch.ops.aten
    targets = (torch.nn.functional.scaled_dot_product_attention, a.scaled_dot_product_attention,
               a.scaled_dot_product_attention.default)
    names = ("query", "key", "value", "attn_mask", "dropout_p", "is_causal", "scale", "enable_gqa")
    graph, count = gm.graph, 0
    for node in list(graph.nodes):
        if node.op != "call_function" or node.target not in targets or len(node.args) < 3:
            continue
        bound = dict(zip(names, node.args))
        bound.update(node.kwargs)
        if bound.get("attn_mask") is not None or bound.get("dropout_p", 0.0) not in (0, 0.0):
            continue
        qkv = [bound["query"], bound["key"], bound["value"]]
        if not all(isinstance(n, fx.Node) for n in qkv):
            continue
        matches = [_match_fp8(n) for n in qkv]
        if any(m is None for m in matches):
            continue
        amaxes = [_const_tensor(gm, m[1]) for m in matches]
        if any(t is not None and t.numel() != 1 for t in amaxes):
            continue
        scale = bound.get("scale")
        if scale is not None and not isinstance(scale, (int, float)):
            continue
        with graph.inserting_before(node):
            out = graph.call_function(torch.ops.tensorrt.b200_fp8_sdpa.default,
                                      (matches[0][0], matches[1][0], matches[2][0], matches[0][1], matches[1][1], matches[2][1],
                                       bool(bound.get("is_causal", False)), float(scale) if scale is not None else -1.0))
        out.meta.update({k: v for k, v in node.meta.items() if k in ("val", "tensor_meta")})
        node.replace_all_uses_with(out)
        graph.erase_node(node)
        for qn in qkv:
            if not qn.users:
                graph.erase_node(qn)
        count += 1
    if count:
        graph.eliminate_dead_code()
        graph.lint()
        gm.recompile()
    return count


def fuse_gated_mlp(gm: fx.GraphModule) -> int:
    """`silu(gate(x)) * up(x)` whose two linears were rewritten by `fuse_quantized_linear` into
    `b200_fp8_gemm` nodes on the SAME quantized activation, with folded (constant) weights and no bias,
    becomes one `tensorrt::b200_fp8_gemm_silu_mul` node on the stacked weight [gate rows; up rows]: the
    activation rides in the GEMM epilogue and the [tokens, 2F] tensor is never written (the bits of the GEMM
    followed by this library's silu * up kernel: one bf16 rounding where eager silu and mul round twice).  This
    is the MLP of the models the reference lowers (`down_proj(act_fn(gate_proj(x)) * up_proj(x))`).  Left
    alone: F not a multiple of 128, weights that are not constants, a bias, an output cast between the GEMM
    and the activation.  When the product feeds nothing but an FP8 quantizer with a constant per-tensor amax,
    that quantizer moves into the epilogue as well (`b200_fp8_gemm_silu_mul_quant` -> codes, scale).  Returns the number of MLPs rewritten; run it after `fuse_quantized_linear`."""
    from . import ops

    ops.load_ops()
    t, a = torch.ops.tensorrt, torch.ops.aten
    gemm = t.b200_fp8_gemm.default
    silus = (torch.nn.functional.silu, a.silu, a.silu.default)
    muls = (operator.mul, torch.mul, a.mul, a.mul.Tensor)
    graph, count = gm.graph, 0
    for node in list(graph.nodes):
        if node.op != "call_function" or node.target not in muls or len(node.args) != 2:
            continue
        lhs, rhs = node.args
        if not (isinstance(lhs, fx.Node) and isinstance(rhs, fx.Node)):
            continue
        act, up = (lhs, rhs) if (lhs.op == "call_function" and lhs.target in silus) else (rhs, lhs)
        if not (act.op == "call_function" and act.target in silus and len(act.args) >= 1 and len(act.users) == 1):
            continue
        gate = act.args[0]
        if not all(isinstance(n, fx.Node) and n.op == "call_function" and n.target is gemm and len(n.users) == 1 for n in (gate, up)):
            continue
        if gate.args[0] is not up.args[0] or gate.args[1] is not up.args[1]:
            continue                                            # not the same quantized activation
        consts = [_const_tensor(gm, n) for n in (gate.args[2], gate.args[3], up.args[2], up.args[3])]
        if any(c is None for c in consts):
            continue
        gc, gs, uc, us = consts
        f = gc.shape[0]
        if gc.shape != uc.shape or f % 128 or gs.numel() not in (1, f) or us.numel() not in (1, f):
            continue
        gs, us = (s_.reshape(-1).expand(f) for s_ in (gs, us))          # a per-tensor scale becomes one per row: same products
        names = []
        for i, stacked in enumerate((torch.cat([gc, uc], dim=0).contiguous(), torch.cat([gs.reshape(-1), us.reshape(-1)]).contiguous())):
            name = f"_b200q_gu{count}_{i}"
            while hasattr(gm, name):
                name += "_"
            gm.register_buffer(name, stacked)
            names.append(name)
        # the product's only reader is an FP8 quantizer with a static per-tensor amax (the calibrated input quantizer
        # of the down projection): it goes into the epilogue too and the node returns (codes, scale) in its place
        quantizer = None
        if len(node.users) == 1:
            user = next(iter(node.users))
            if user.op == "call_function" and user.target is t.b200_fp8_quantize.default and len(user.args) == 2 and user.args[0] is node:
                amax_const = _const_tensor(gm, user.args[1])
                if amax_const is not None and amax_const.numel() == 1:
                    quantizer = user
        with graph.inserting_before(quantizer if quantizer is not None else node):
            w_parts = [graph.get_attr(n) for n in names]
            if quantizer is not None:
                out = graph.call_function(t.b200_fp8_gemm_silu_mul_quant.default, (gate.args[0], gate.args[1], *w_parts, quantizer.args[1]))
            else:
                out = graph.call_function(t.b200_fp8_gemm_silu_mul.default, (gate.args[0], gate.args[1], *w_parts))
        if quantizer is not None:
            quantizer.replace_all_uses_with(out)
            graph.erase_node(quantizer)
        else:
            out.meta.update({k: v for k, v in node.meta.items() if k in ("val", "tensor_meta")})
            node.replace_all_uses_with(out)
        old_consts = [gate.args[2], gate.args[3], up.args[2], up.args[3]]
        for dead in (node, act, gate, up):
            if not dead.users:
                graph.erase_node(dead)
        for c in old_consts:
            _drop_unused_constant(gm, c)
        count += 1
    if count:
        graph.eliminate_dead_code()
        graph.lint()
        gm.recompile()
    return count


def fuse_all_reduce_wait(gm: fx.GraphModule) -> int:
    """`_c10d_functional.all_reduce(x, op, group)` whose only user is `wait_tensor` becomes one
    `tensorrt::fused_nccl_all_reduce(x, op, group)` node, the form the reference's converters (and
    this package's row-parallel paths) consume
    (py/torch_tensorrt/dynamo/lowering/passes/fuse_distributed_ops.py:167-234).  An all-reduce whose
    result is used by anything besides a single wait is left alone.  Returns the number of pairs
    fused; the module is recompiled in place."""
    from . import ops

    ops.load_ops()
    c10d = torch.ops._c10d_functional
    fused_op = torch.ops.tensorrt.fused_nccl_all_reduce.default
    graph, count = gm.graph, 0
    for node in list(graph.nodes):
        if node.op != "call_function" or node.target is not c10d.all_reduce.default or len(node.users) != 1:
            continue
        wait = next(iter(node.users))
        if wait.op != "call_function" or wait.target is not c10d.wait_tensor.default:
            continue
        with graph.inserting_after(wait):
            fused = graph.call_function(fused_op, tuple(node.args[:3]))
        fused.meta.update(node.meta)
        wait.replace_all_uses_with(fused)
        graph.erase_node(wait)
        graph.erase_node(node)
        count += 1
    if count:
        graph.eliminate_dead_code()
        graph.lint()
        gm.recompile()
    return count
