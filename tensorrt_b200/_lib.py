"""ctypes binding of the b200q C ABI (include/b200q.h).

The library is loaded from the package directory; when it is missing it is built in
place (nvcc required).  There is no fallback implementation: a missing or unloadable
library is an error.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

from . import _build

_c = ctypes
_i64 = _c.c_int64
_p = _c.c_void_p

# name -> (restype, argtypes); kept in the order of include/b200q.h
SIGNATURES = {
    "b200q_version": (_c.c_int, []),
    "b200q_status_string": (_c.c_char_p, [_c.c_int]),
    "b200q_amax_workspace_bytes": (_c.c_size_t, []),
    "b200q_amax": (_c.c_int, [_p, _c.c_int, _i64, _p, _p, _c.c_size_t, _p]),
    "b200q_row_amax": (_c.c_int, [_p, _c.c_int, _i64, _i64, _p, _p]),
    "b200q_amax_static_max_elements": (_i64, []),
    "b200q_amax_static": (_c.c_int, [_p, _c.c_int, _i64, _p, _p]),
    "b200q_fp8_quantize": (_c.c_int, [_p, _c.c_int, _i64, _i64, _p, _i64, _p, _p, _p]),
    "b200q_fp8_fake_quantize": (_c.c_int, [_p, _c.c_int, _i64, _i64, _p, _i64, _p, _p]),
    "b200q_fp8_dequantize": (_c.c_int, [_p, _p, _i64, _i64, _i64, _p, _c.c_int, _p]),
    "b200q_nvfp4_scale_bytes": (_c.c_size_t, [_i64, _i64]),
    "b200q_nvfp4_quantize": (_c.c_int, [_p, _c.c_int, _i64, _i64, _p, _p, _p, _p, _p]),
    "b200q_nvfp4_fake_quantize": (_c.c_int, [_p, _c.c_int, _i64, _i64, _p, _p, _p]),
    "b200q_nvfp4_dequantize": (_c.c_int, [_p, _p, _p, _i64, _i64, _p, _c.c_int, _p]),
    "b200q_fp8_gemm": (_c.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _p, _p]),
    "b200q_fp8_gemm_silu_mul": (_c.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _p, _p]),
    "b200q_fp8_gemm_silu_mul_quantize": (_c.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _p, _p, _i64, _i64, _i64, _p, _p]),
    "b200q_nvfp4_gemm": (_c.c_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _p]),
    "b200q_fp8_gemm_reduce_scatter": (_c.c_int, [_p, _p, _i64, _p, _p, _i64, _p, _i64, _i64, _i64, _p, _p]),
    "b200q_nvfp4_gemm_reduce_scatter": (_c.c_int, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _p]),
    "b200q_comm_create": (_c.c_int, [_c.c_int, _c.c_int, _p, _p, _p]),
    "b200q_comm_alloc": (_c.c_int, [_p, _c.c_size_t, _p]),
    "b200q_comm_destroy": (_c.c_int, [_p]),
    "b200q_reduce_gather": (_c.c_int, [_p, _p, _i64, _i64, _c.c_uint32, _p, _p]),
    "b200q_reduce_add_gather": (_c.c_int, [_p, _p, _p, _i64, _i64, _c.c_uint32, _p, _p]),
    "b200q_reduce_add_rms_norm_fp8_quantize_gather": (_c.c_int, [_p, _p, _p, _p, _c.c_float, _i64, _i64, _c.c_uint32, _p, _p]),
    "b200q_pull_signal": (_c.c_int, [_p, _p]),
    "b200q_pull_reduce_add_rms_norm_fp8_quantize": (_c.c_int, [_p, _p, _p, _p, _c.c_float, _p, _p, _i64, _i64, _p, _p]),
    "b200q_pull_reduce_add": (_c.c_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "b200q_fp8_quantize_transpose": (_c.c_int, [_p, _c.c_int, _i64, _i64, _i64, _p, _p, _i64, _p, _p]),
    "b200q_fp8_sdpa": (_c.c_int, [_p, _p, _p, _p, _p, _p, _p, _c.c_int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _c.c_float, _c.c_int, _p]),
    "b200q_rms_norm": (_c.c_int, [_p, _p, _p, _i64, _i64, _c.c_float, _p]),
    "b200q_add_rms_norm_fp8_quantize": (_c.c_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _c.c_float, _p]),
    "b200q_silu_mul": (_c.c_int, [_p, _p, _i64, _i64, _p]),
    "b200q_silu_mul_fp8_quantize": (_c.c_int, [_p, _p, _p, _i64, _i64, _p]),
    "b200q_add": (_c.c_int, [_p, _p, _p, _i64, _p]),
    "b200q_expand_heads": (_c.c_int, [_p, _i64, _i64, _p, _i64, _c.c_int, _c.c_int, _c.c_int, _p]),
    "b200q_expand_heads_fp8_quantize": (_c.c_int, [_p, _i64, _i64, _p, _p, _i64, _c.c_int, _c.c_int, _c.c_int, _p]),
    "b200q_device_status": (_c.c_int, [_c.c_int]),
}



class Cfg(ctypes.Structure):
    """struct b200q_cfg of include/b200q.h: per-call options (NULL = defaults)."""
    _fields_ = [("tile_n", _c.c_int32), ("static_weights", _c.c_int32), ("peer_wait_ms", _c.c_uint32), ("reserved", _c.c_uint32)]


def cfg_ref(tile_n: int = 0, static_weights: bool = False, peer_wait_ms: int = 0):
    """ctypes reference to a b200q_cfg, or None (NULL) when every field has its default."""
    if not tile_n and not static_weights and not peer_wait_ms:
        return None
    return ctypes.byref(Cfg(int(tile_n), 1 if static_weights else 0, int(peer_wait_ms), 0))


class Peers(ctypes.Structure):
    """struct b200q_peers of include/b200q.h."""
    _fields_ = [("rank", _c.c_int32), ("world", _c.c_int32), ("recv", _p * 8), ("out", _p * 8), ("flags", _p * 8)]


class GatherPeers(ctypes.Structure):
    """struct b200q_gather_peers of include/b200q.h."""
    _fields_ = [("rank", _c.c_int32), ("world", _c.c_int32), ("recv", _p * 8), ("codes", _p * 8), ("scales", _p * 8),
                ("flags", _p * 8)]


ALLGATHER_FN = ctypes.CFUNCTYPE(_c.c_int, _p, _p, _p, _c.c_size_t)   # b200q_allgather_fn


class PullPeers(ctypes.Structure):
    """struct b200q_pull_peers of include/b200q.h."""
    _fields_ = [("rank", _c.c_int32), ("world", _c.c_int32), ("partial", _p * 8), ("flags", _p * 8)]


_lib = None


def header_symbols() -> list[str]:
    """Every function name declared in include/b200q.h."""
    text = (_build.ROOT / "include" / "b200q.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = Path(_build.LIB)
    if not path.exists():
        _build.build_cuda()
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class B200QError(RuntimeError):
    def __init__(self, status: int, what: str):
        msg = load().b200q_status_string(status).decode()
        super().__init__(f"{what} failed: {msg} (status {status})")
        self.status = status


def check(status: int, what: str) -> None:
    if status != 0:
        raise B200QError(status, what)
