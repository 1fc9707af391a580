"""CPU checks of the native boundary: the C-ABI library loads and exports every symbol the
header declares; argument validation that needs no device; the torch ops' schemas and
fake kernels; export of a Q/DQ linear; plugin registration against a fake `custom_op`."""
import ctypes

import pytest
import torch


def test_every_header_symbol_is_exported(b200):
    from tensorrt_b200 import _lib

    lib = _lib.load()
    names = _lib.header_symbols()
    assert len(names) >= 16
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/b200q.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table out of step with the header"


def test_status_strings_and_sizes(b200):
    from tensorrt_b200 import _lib

    lib = _lib.load()
    assert lib.b200q_version() >= 100
    assert lib.b200q_status_string(0) == b"ok"
    for code in range(-7, 0):
        assert lib.b200q_status_string(code) not in (b"ok", b"unknown status")
    assert lib.b200q_nvfp4_scale_bytes(8192, 8192) == 8192 * 8192 // 16
    assert lib.b200q_nvfp4_scale_bytes(300, 37 * 16) == 3 * 10 * 512
    assert lib.b200q_nvfp4_scale_bytes(0, 64) == 0
    assert lib.b200q_amax_workspace_bytes() >= 148 * 8 * 4


def test_argument_validation_without_a_device(b200):
    """Shape / pointer checks come before any CUDA call, so they can run here."""
    from tensorrt_b200 import _lib

    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 255) & ~255
    assert lib.b200q_fp8_quantize(None, 2, 4, 64, p, 1, p, p, None) == -1          # null input
    assert lib.b200q_fp8_quantize(p, 7, 4, 64, p, 1, p, p, None) == -1             # bad dtype
    assert lib.b200q_fp8_quantize(p, 2, 4, 24, p, 1, p, p, None) == -1             # cols % 16
    assert lib.b200q_fp8_quantize(p, 2, 4, 64, p, 3, p, p, None) == -1             # amax_numel not 0/1/rows
    assert lib.b200q_fp8_quantize(p + 2, 2, 4, 64, p, 1, p, p, None) == -2         # misaligned
    assert lib.b200q_nvfp4_quantize(p, 2, 4, 40, p, p, p, p, None) == -1           # cols % 16
    assert lib.b200q_nvfp4_gemm(p, p, p, p, p, p, None, p, 4, 4, 48, None, None) == -1   # K % 32
    assert lib.b200q_fp8_gemm(p, p, 1, p, p, 1, None, p, 4, 4, 40, None, None) == -1     # K % 16
    assert lib.b200q_fp8_gemm(p, p, 3, p, p, 1, None, p, 4, 4, 64, None, None) == -1     # scale count
    assert lib.b200q_amax(p, 2, 64, p, None, 0, None) == -5                         # no workspace
    # per-call options: an unknown tile selector or a non-zero reserved field is refused before any CUDA call
    for tile in (64, 1003, -1):
        assert lib.b200q_fp8_gemm(p, p, 1, p, p, 1, None, p, 4, 4, 64, None, _lib.cfg_ref(tile_n=tile)) == -1
        assert lib.b200q_nvfp4_gemm(p, p, p, p, p, p, None, p, 4, 4, 64, None, _lib.cfg_ref(tile_n=tile)) == -1
    bad = _lib.Cfg(0, 0, 0, 7)
    assert lib.b200q_fp8_gemm(p, p, 1, p, p, 1, None, p, 4, 4, 64, None, ctypes.byref(bad)) == -1
    assert _lib.cfg_ref() is None and ctypes.sizeof(_lib.Cfg) == 16


def test_the_abi_has_no_process_wide_setter(b200):
    """Tile choice, the static-weights promise and the peer wait limit travel per call in
    b200q_cfg; nothing in the header sets state for later calls."""
    from tensorrt_b200 import _lib

    assert not [n for n in _lib.header_symbols() if "_set_" in n or n.endswith("_assume_static_weights")]


def test_validation_of_the_fused_and_peer_entry_points_without_a_device(b200):
    from tensorrt_b200 import _lib

    lib = _lib.load()
    buf = ctypes.create_string_buffer(8192)
    p = (ctypes.addressof(buf) + 255) & ~255
    assert lib.b200q_silu_mul_fp8_quantize(None, p, p, 4, 64, None) == -1           # null input
    assert lib.b200q_silu_mul_fp8_quantize(p, p, p, 4, 60, None) == -1              # f % 8
    assert lib.b200q_silu_mul_fp8_quantize(p, p, p, 4, 32776, None) == -1           # f beyond 32768
    assert lib.b200q_silu_mul_fp8_quantize(p, p, p, 0, 64, None) == 0               # empty: no-op
    assert lib.b200q_silu_mul_fp8_quantize(p + 2, p, p, 4, 64, None) == -2          # misaligned
    assert lib.b200q_add_rms_norm_fp8_quantize(p, None, p, None, p, p, 4, 16392, 1e-5, None) == -1   # cols beyond 16384
    peers = _lib.Peers()
    peers.rank, peers.world = 0, 2
    for r in range(2):
        peers.recv[r], peers.out[r], peers.flags[r] = p, p, p
    ref = ctypes.byref(peers)
    assert lib.b200q_reduce_gather(None, None, 256, 64, 1, None, None) == -1               # no peers
    assert lib.b200q_reduce_gather(ref, None, 200, 64, 1, None, None) == -1                # M not a multiple of world * 128
    assert lib.b200q_reduce_gather(ref, None, 256, 60, 1, None, None) == -1                # N % 8
    assert lib.b200q_reduce_add_gather(ref, None, None, 256, 64, 1, None, None) == -1      # residual shard is required
    assert lib.b200q_fp8_gemm_reduce_scatter(p, p, 1, p, p, 1, ref, 200, 64, 64, None, None) == -1   # M not a multiple of world * 128
    peers.world = 9
    assert lib.b200q_reduce_gather(ref, None, 9 * 128, 64, 1, None, None) == -1            # more than 8 ranks
    gp = _lib.GatherPeers()
    gp.rank, gp.world = 1, 2
    for r in range(2):
        gp.recv[r], gp.codes[r], gp.scales[r], gp.flags[r] = p, p, p, p
    gref = ctypes.byref(gp)
    f = lib.b200q_reduce_add_rms_norm_fp8_quantize_gather
    assert f(gref, None, None, p, 1e-5, 256, 64, 1, None, None) == -1                      # no residual shard
    assert f(gref, None, p, None, 1e-5, 256, 64, 1, None, None) == -1                      # no norm weight
    assert f(gref, None, p, p, 1e-5, 256, 72, 1, None, None) == -1                         # N % 16
    assert f(gref, None, p, p, 1e-5, 256, 16400, 1, None, None) == -1                      # N beyond 16384
    assert f(gref, None, p, p, 1e-5, 384, 64, 1, None, None) == -1                         # M not a multiple of world * 128
    gp.codes[1] = None
    assert f(gref, None, p, p, 1e-5, 256, 64, 1, None, None) == -1                         # a peer buffer is missing


def test_product_does_not_reach_into_test_infrastructure():
    """Nothing under the package may import, read or run the oracle or scratch files."""
    import pathlib
    import re

    root = pathlib.Path(__file__).resolve().parents[1]
    bad = re.compile(r"^\s*(from|import)\s+(oracle|_work)\b|['\"/]_work/|['\"/]oracle/")
    for path in list((root / "tensorrt_b200").rglob("*.py")) + list((root / "tensorrt_b200" / "csrc").glob("*")) + [root / "include" / "b200q.h"]:
        if path.is_file() and path.suffix in (".py", ".cu", ".cuh", ".h", ".cpp"):
            for n, line in enumerate(path.read_text().splitlines(), 1):
                assert not bad.search(line), f"{path}:{n}: {line.strip()}"


def test_product_has_no_cpu_path(b200):
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        b200.capi.fp8_quantize(torch.randn(4, 64))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        b200.capi.nvfp4_quantize(torch.randn(4, 64), torch.tensor(1.0))
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.tensorrt.quantize_op(torch.randn(4, 64), torch.tensor(1.0), 8, 4, False, False)


def test_op_schemas_match_the_reference_call_sites(b200):
    q = torch.ops.tensorrt.quantize_op.default._schema
    assert [a.name for a in q.arguments][:2] == ["input", "amax"]
    assert [str(a.type) for a in q.arguments] == ["Tensor", "Tensor", "int", "int", "bool", "bool"]
    d = torch.ops.tensorrt.dynamic_block_quantize_op.default._schema
    assert [str(a.type) for a in d.arguments] == ["Tensor", "int", "Tensor", "int", "int", "int", "int"]
    r = torch.ops.tensorrt.fused_nccl_all_reduce.default._schema
    assert [str(a.type) for a in r.arguments] == ["Tensor", "str", "str"]
    assert len(r.arguments) == 3


def test_meta_kernels_shapes_and_dtypes(b200):
    x = torch.empty(3, 5, 64, device="meta", dtype=torch.bfloat16)
    a = torch.empty((), device="meta")
    assert torch.ops.tensorrt.quantize_op(x, a, 8, 4, False, False).shape == x.shape
    y = torch.ops.tensorrt.dynamic_block_quantize_op(x, 16, a, 4, 2, 8, 4)
    assert y.shape == x.shape and y.dtype == x.dtype
    codes, scales = torch.ops.tensorrt.b200_fp8_quantize(x, None)
    assert codes.shape == x.shape and codes.dtype == torch.uint8 and scales.shape == (15,)
    codes, sf, g = torch.ops.tensorrt.b200_nvfp4_quantize(x, a)
    assert codes.shape == (3, 5, 32) and sf.shape == (512,) and g.shape == ()
    w = torch.empty(128, 64, device="meta", dtype=torch.uint8)
    xc, xs, ws = torch.empty(3, 5, 64, device="meta", dtype=torch.uint8), torch.empty(15, device="meta"), torch.empty(128, device="meta")
    bias = torch.empty(128, device="meta", dtype=torch.bfloat16)
    for out in (torch.ops.tensorrt.b200_fp8_gemm(xc, xs, w, ws), torch.ops.tensorrt.b200_fp8_gemm_bias(xc, xs, w, ws, bias)):
        assert out.shape == (3, 5, 128) and out.dtype == torch.bfloat16
    # one-node linears: the result has the activation's shape prefix and dtype
    for dt in (torch.bfloat16, torch.float16):
        xa = torch.empty(3, 5, 64, device="meta", dtype=dt)
        for out in (torch.ops.tensorrt.b200_fp8_linear(xa, a, w, ws), torch.ops.tensorrt.b200_fp8_linear_bias(xa, a, w, ws, bias)):
            assert out.shape == (3, 5, 128) and out.dtype == dt
        w4, s4 = torch.empty(128, 32, device="meta", dtype=torch.uint8), torch.empty(512, device="meta", dtype=torch.uint8)
        for out in (torch.ops.tensorrt.b200_nvfp4_linear(xa, a, w4, s4, a), torch.ops.tensorrt.b200_nvfp4_linear_bias(xa, a, w4, s4, a, bias)):
            assert out.shape == (3, 5, 128) and out.dtype == dt


def test_export_keeps_quantize_nodes(b200):
    """A Q/DQ-wrapped linear traced with fake tensors keeps both quantize ops as nodes, as the
    reference needs (its constant folder marks them impure so they are never folded away)."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.fx.experimental.proxy_tensor import make_fx

    def f(x, w, ax, aw):
        xq = torch.ops.tensorrt.quantize_op(x, ax, 8, 4, False, False)
        wq = torch.ops.tensorrt.dynamic_block_quantize_op(w, 16, aw, 4, 2, 8, 4)
        return torch.nn.functional.linear(xq, wq)

    with FakeTensorMode(allow_non_fake_inputs=True) as mode:
        args = [mode.from_tensor(torch.empty(*s, device="meta", dtype=torch.bfloat16)) for s in ((8, 64), (32, 64))]
        args += [mode.from_tensor(torch.empty((), device="meta")) for _ in range(2)]
        gm = make_fx(f)(*args)
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert torch.ops.tensorrt.quantize_op.default in targets
    assert torch.ops.tensorrt.dynamic_block_quantize_op.default in targets


def _generator_like_custom_op(calls):
    """A stand-in for torch_tensorrt's `plugins.custom_op` that applies the rules of its generator
    (py/torch_tensorrt/dynamo/conversion/plugins/_generate_plugin.py:113-185, 196-270;
    _generate_plugin_converter.py:126,143) to the op it is given:
      - every argument type must be exactly Tensor, float, int, bool or str ("arg type is not handled");
      - tensor arguments come before all others (the converter slices `args[0:len(tensor_inputs)]`);
      - the fake kernel is run on float32 fake tensors with symbolic sizes for every tensor argument;
      - every output descriptor is `tensor_args[0].like()`: the output dtype is the first tensor
        argument's, which must agree with what the op's fake kernel returns for real dtypes."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.fx.experimental.symbolic_shapes import DimDynamic, ShapeEnv

    def custom_op(name, capability_validator=None, priority=None, supports_dynamic_shapes=False,
                  requires_output_allocator=False, *, use_aot_if_available=True, _aot_register=None):
        ns, op = name.split("::")
        packet = getattr(getattr(torch.ops, ns), op)
        schema = packet._schemas[""]
        kinds = [str(a.type) for a in schema.arguments]
        for k in kinds:
            if k not in ("Tensor", "float", "int", "bool", "str"):
                raise ValueError("arg type is not handled")
        n_tensors = sum(k == "Tensor" for k in kinds)
        assert all(k == "Tensor" for k in kinds[:n_tensors]), f"{name}: a tensor argument follows a scalar"
        scalars = {"int": 16, "float": 1.0, "bool": False, "str": "sum"}
        scalar_args = {"tensorrt::quantize_op": [8, 4, False, False],
                       "tensorrt::b200_dynamic_block_quantize_tensors_first": [16, 4, 2, 8, 4]}.get(name, [scalars[k] for k in kinds[n_tensors:]])
        shape_env = ShapeEnv()
        with FakeTensorMode(shape_env=shape_env):
            fake_args = []
            for i in range(n_tensors):
                # amax-like arguments are scalars in every call site; the rest get 2-D symbolic shapes
                arg = schema.arguments[i].name
                if "amax" in arg or "global" in arg:
                    fake_args.append(torch.randn(()))
                elif "scales" in arg or arg == "bias":
                    fake_args.append(torch.randn(64))
                else:
                    fake_args.append(torch.randn(64, 64))
            out = packet(*fake_args, *scalar_args)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        assert len(outs) == len(schema.returns)
        for o in outs:
            assert o.dtype == fake_args[0].dtype, f"{name}: output dtype {o.dtype} is not the first tensor argument's"
        calls.append((name, priority, supports_dynamic_shapes))

    return custom_op


def test_plugin_registration_against_the_generator_rules(b200):
    calls, converters = [], {}

    def decorator(target, *, priority=None, supports_dynamic_shapes=False, **kw):
        def reg(fn):
            converters[target] = (fn, priority, supports_dynamic_shapes)
            return fn
        return reg

    seen = {}

    def lookup(overload):
        def impl(ctx, target, args, kwargs, name):
            seen["call"] = (target, args, kwargs, name)
            return "layer-output"
        return impl

    names = b200.register_with_torch_tensorrt(custom_op=_generator_like_custom_op(calls), priority="HIGH",
                                              converter_decorator=decorator, lookup=lookup)
    assert "tensorrt::quantize_op" in names and "tensorrt::b200_fp8_linear_bias" in names and "tensorrt::b200_nvfp4_linear" in names
    assert names[-1] == "tensorrt::dynamic_block_quantize_op"
    assert all(p == "HIGH" and dyn for _, p, dyn in calls)
    # the hand-written converter sits on the ORIGINAL target at HIGH priority and forwards with amax moved forward
    target = torch.ops.tensorrt.dynamic_block_quantize_op.default
    fn, prio, dyn = converters[target]
    assert prio == "HIGH" and dyn
    assert fn(None, target, ("x", 16, "amax", 4, 2, 8, 4), {}, "node7") == "layer-output"
    alias = torch.ops.tensorrt.b200_dynamic_block_quantize_tensors_first.default
    assert seen["call"] == (alias, ("x", "amax", 16, 4, 2, 8, 4), {}, "node7")
    assert fn(None, target, ("x", 16, "amax"), {"num_bits": 4, "exponent_bits": 2, "scale_num_bits": 8, "scale_exponent_bits": 4},
              "n") == "layer-output"
    with pytest.raises(ValueError):
        fn(None, target, ("x", 16), {}, "n")


def test_the_generator_rules_reject_what_the_real_generator_rejects(b200):
    """The stand-in is only worth something if it fails where the real one would: an optional
    tensor argument, and an op whose output dtype differs from its first tensor argument's."""
    custom_op = _generator_like_custom_op([])
    with pytest.raises(ValueError, match="arg type is not handled"):
        custom_op("tensorrt::b200_fp8_quantize")            # (Tensor input, Tensor? amax)
    with pytest.raises(AssertionError, match="output dtype"):
        custom_op("tensorrt::b200_fp8_gemm")                # bf16 out of uint8 codes
    with pytest.raises(AssertionError, match="follows a scalar"):
        custom_op("tensorrt::dynamic_block_quantize_op")    # (input, block_size, amax, ...)


def test_registration_is_a_logged_no_op_without_torch_tensorrt(b200):
    try:
        import torch_tensorrt  # noqa: F401
    except Exception:
        assert b200.register_with_torch_tensorrt() == []


def test_comm_context_argument_validation():
    """b200q_comm_create rejects impossible rank / world values before touching a device."""
    import ctypes

    from tensorrt_b200 import _lib

    lib = _lib.load()
    h = ctypes.c_void_p()
    null_cb = _lib.ALLGATHER_FN(0)
    for rank, world in [(-1, 2), (2, 2), (0, 0), (0, 9)]:
        assert lib.b200q_comm_create(rank, world, null_cb, None, ctypes.byref(h)) == -1
    assert lib.b200q_comm_create(0, 2, null_cb, None, ctypes.byref(h)) == -1     # several ranks need the all-gather
    assert lib.b200q_comm_create(0, 1, null_cb, None, None) == -1
    assert lib.b200q_comm_alloc(None, 16, (ctypes.c_void_p * 8)()) == -1
    assert lib.b200q_comm_destroy(None) == 0


def test_validation_of_the_fused_gate_up_gemm_without_a_device(b200):
    """b200q_fp8_gemm_silu_mul[_quantize]: argument errors are reported before anything touches a device."""
    from tensorrt_b200 import _lib

    lib = _lib.load()
    buf = ctypes.create_string_buffer(8192)
    p = (ctypes.addressof(buf) + 255) & ~255
    f, g = lib.b200q_fp8_gemm_silu_mul, lib.b200q_fp8_gemm_silu_mul_quantize
    assert f(None, p, 1, p, p, 1, None, p, 256, 256, 64, None, None) == -1           # null operand
    assert f(p, p, 1, p, p, 1, None, p, 256, 384, 64, None, None) == -1              # N = 2F with F not a multiple of 128
    assert f(p, p, 1, p, p, 1, None, p, 256, 256, 72, None, None) == -1              # K % 16
    assert f(p, p, 7, p, p, 1, None, p, 256, 256, 64, None, None) == -1              # activation scales: 1 or M
    assert f(p + 4, p, 1, p, p, 1, None, p, 256, 256, 64, None, None) == -2          # misaligned codes
    cfg = _lib.Cfg()
    cfg.tile_n = 128
    assert f(p, p, 1, p, p, 1, None, p, 256, 256, 64, None, ctypes.byref(cfg)) == -1  # one kernel serves this entry: no tile choice
    assert g(p, p, 1, p, p, 1, None, None, p, p, 256, 256, 64, None, None) == -1     # the static amax is required
    assert g(p, p, 1, p, p, 1, None, p, None, p, 256, 256, 64, None, None) == -1     # so is the code buffer
    assert g(p, p, 1, p, p, 1, None, p, p, None, 256, 384, 64, None, None) == -1     # F not a multiple of 128
