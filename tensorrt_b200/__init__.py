"""B200-native (sm_100a) quantized-linear hot path behind Torch-TensorRT's operator API.

    import tensorrt_b200                      # loads the native libraries, registers tensorrt::* ops
    torch.ops.tensorrt.quantize_op(x, amax, 8, 4, False, False)            # FP8 fake-quant (eager semantics)
    torch.ops.tensorrt.dynamic_block_quantize_op(x, 16, amax, 4, 2, 8, 4)  # NVFP4 fake-quant
    tensorrt_b200.Fp8Linear.from_float(linear)(x)                           # real-quant FP8 GEMM path
    tensorrt_b200.Nvfp4Linear.from_float(linear)(x)                         # real-quant NVFP4 GEMM path
    tensorrt_b200.fuse_quantized_linear(graph_module)                       # Q/DQ-wrapped linears -> GEMM nodes
    tensorrt_b200.fuse_gated_mlp(graph_module)                              # silu(gate(x)) * up(x) -> one GEMM

Only CUDA (compute capability 10.x) is implemented; there is no CPU or other-GPU fallback.
"""
from . import capi  # noqa: F401
from ._lib import B200QError, load as load_library  # noqa: F401
from .ops import load_ops, ops_loaded  # noqa: F401
from .linear import Fp8GatedMlp, Fp8Linear, Nvfp4Linear, QuantizedLinear, fp8_linear, nvfp4_linear  # noqa: F401
from .plugin import register_with_torch_tensorrt  # noqa: F401
from .fx_passes import fuse_all_reduce_wait, fuse_fp8_sdpa, fuse_gated_mlp, fuse_quantized_linear  # noqa: F401

__all__ = ["capi", "B200QError", "load_library", "load_ops", "ops_loaded", "Fp8GatedMlp", "Fp8Linear", "Nvfp4Linear",
           "QuantizedLinear", "fp8_linear", "nvfp4_linear", "register_with_torch_tensorrt", "fuse_quantized_linear", "fuse_all_reduce_wait", "fuse_fp8_sdpa", "fuse_gated_mlp"]

load_ops()
