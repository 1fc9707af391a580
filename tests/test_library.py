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
    assert lib.b200q_nvfp4_gemm(p, p, p, p, p, p, None, p, 4, 4, 48, None) == -1   # K % 32
    assert lib.b200q_fp8_gemm(p, p, 1, p, p, 1, None, p, 4, 4, 40, None) == -1     # K % 16
    assert lib.b200q_fp8_gemm(p, p, 3, p, p, 1, None, p, 4, 4, 64, None) == -1     # scale count
    assert lib.b200q_amax(p, 2, 64, p, None, 0, None) == -5                         # no workspace
    assert lib.b200q_gemm_set_tile_n(64) == -1
    assert lib.b200q_gemm_set_tile_n(1003) == -1
    assert lib.b200q_gemm_set_tile_n(0) == 0


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
    assert lib.b200q_reduce_gather(None, None, 256, 64, 1, None) == -1               # no peers
    assert lib.b200q_reduce_gather(ref, None, 200, 64, 1, None) == -1                # M not a multiple of world * 128
    assert lib.b200q_reduce_gather(ref, None, 256, 60, 1, None) == -1                # N % 8
    assert lib.b200q_reduce_add_gather(ref, None, None, 256, 64, 1, None) == -1      # residual shard is required
    peers.world = 9
    assert lib.b200q_reduce_gather(ref, None, 9 * 128, 64, 1, None) == -1            # more than 8 ranks
    gp = _lib.GatherPeers()
    gp.rank, gp.world = 1, 2
    for r in range(2):
        gp.recv[r], gp.codes[r], gp.scales[r], gp.flags[r] = p, p, p, p
    gref = ctypes.byref(gp)
    f = lib.b200q_reduce_add_rms_norm_fp8_quantize_gather
    assert f(gref, None, None, p, 1e-5, 256, 64, 1, None) == -1                      # no residual shard
    assert f(gref, None, p, None, 1e-5, 256, 64, 1, None) == -1                      # no norm weight
    assert f(gref, None, p, p, 1e-5, 256, 72, 1, None) == -1                         # N % 16
    assert f(gref, None, p, p, 1e-5, 256, 16400, 1, None) == -1                      # N beyond 16384
    assert f(gref, None, p, p, 1e-5, 384, 64, 1, None) == -1                         # M not a multiple of world * 128
    gp.codes[1] = None
    assert f(gref, None, p, p, 1e-5, 256, 64, 1, None) == -1                         # a peer buffer is missing


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
    out = torch.ops.tensorrt.b200_fp8_gemm(torch.empty(3, 5, 64, device="meta", dtype=torch.uint8),
                                           torch.empty(15, device="meta"), w, torch.empty(128, device="meta"), None)
    assert out.shape == (3, 5, 128) and out.dtype == torch.bfloat16


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


def test_plugin_registration_with_fake_custom_op(b200):
    calls = []

    def fake_custom_op(name, capability_validator=None, priority=None, supports_dynamic_shapes=False,
                       requires_output_allocator=False):
        ns, op = name.split("::")
        overload = getattr(getattr(torch.ops, ns), op).default
        schema = overload._schema
        # the generated converter slices tensors first, scalars after
        kinds = [str(a.type) for a in schema.arguments]
        first_scalar = next((i for i, k in enumerate(kinds) if not k.startswith("Tensor")), len(kinds))
        assert all(not k.startswith("Tensor") for k in kinds[first_scalar:]), f"{name}: tensor after scalar"
        calls.append((name, priority, supports_dynamic_shapes))

    names = b200.register_with_torch_tensorrt(custom_op=fake_custom_op, priority="HIGH")
    assert "tensorrt::quantize_op" in names
    assert any("dynamic_block_quantize" in n for n in names)
    assert all(p == "HIGH" and dyn for _, p, dyn in calls)
    # without torch_tensorrt installed the real registration is a logged no-op
    try:
        import torch_tensorrt  # noqa: F401
    except Exception:
        assert b200.register_with_torch_tensorrt() == []
