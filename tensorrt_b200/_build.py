"""In-tree build of the native libraries.

`libb200q.so`      — CUDA kernels + the C ABI declared in include/b200q.h (nvcc, sm_100a only).
`libb200q_torch.so` — the torch.library shim registering the `tensorrt::` ops on top of it (g++).

Both are written next to this file so they travel with the source tree; nothing is
installed into site-packages and no JIT cache is used.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
ROOT = PKG.parent
LIB = PKG / "libb200q.so"
TORCH_LIB = PKG / "libb200q_torch.so"

CUDA_SOURCES = ["runtime.cu", "quantize_fp8.cu", "quantize_nvfp4.cu", "gemm_fp8.cu", "gemm_nvfp4.cu",
                "fused_ops.cu", "p2p_allreduce.cu", "attention_fp8.cu", "comm_context.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the b200q kernels cannot be built")


def _stamp(paths, extra="") -> str:
    # content + file name only: the stamp must not change when the tree is copied elsewhere
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths, key=lambda q: Path(q).name):
        h.update(Path(p).name.encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


class _BuildLock:
    """Inter-process lock: ranks of one job importing the package at the same time must not
    compile into the same files concurrently."""

    def __enter__(self):
        import fcntl

        (PKG / "build").mkdir(exist_ok=True)
        self.f = open(PKG / "build" / ".lock", "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl

        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def _run(cmd, log_path: Path | None = None) -> str:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path is not None:
        log_path.write_text(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ...")
    return proc.stdout


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ for sm_100a and link libb200q.so."""
    with _BuildLock():
        return _build_cuda(force, verbose)


def _build_cuda(force: bool, verbose: bool) -> Path:
    sources = [CSRC / s for s in CUDA_SOURCES if (CSRC / s).exists()]
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [ROOT / "include" / "b200q.h"]
    stamp = _stamp(sources + headers, " ".join(NVCC_FLAGS))
    stamp_file = PKG / "build" / "cuda.stamp"
    if not force and LIB.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LIB
    (PKG / "build").mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources:
        obj = PKG / "build" / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(ROOT / "include"), "-c", str(src), "-o", str(obj)]
        procs.append((src, cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, cmd, p in procs:
        out, _ = p.communicate()
        (PKG / "build" / (src.stem + ".ptxas.log")).write_text(" ".join(cmd) + "\n" + out)
        if verbose:
            sys.stderr.write(out)
        if p.returncode != 0:
            sys.stderr.write(out)
            failed = True
    if failed:
        raise RuntimeError("nvcc failed")
    _run([nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-ldl"])
    stamp_file.write_text(stamp)
    return LIB


def build_torch_shim(force: bool = False) -> Path:
    """Compile the torch.library shim (C++17, no CUDA code) against libb200q.so."""
    with _BuildLock():
        return _build_torch_shim(force)


def _build_torch_shim(force: bool) -> Path:
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch_ops.cpp"
    stamp = _stamp([src, ROOT / "include" / "b200q.h"], torch.__version__)
    stamp_file = PKG / "build" / "torch.stamp"
    if not force and TORCH_LIB.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return TORCH_LIB
    (PKG / "build").mkdir(exist_ok=True)
    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-isystem", p]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc += ["-isystem", f"{cuda_home}/include"]
    torch_lib = Path(torch.__file__).parent / "lib"
    cxx11 = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}",
           "-I", str(ROOT / "include"), *inc, str(src), "-o", str(TORCH_LIB),
           f"-L{PKG}", "-lb200q", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           f"-L{cuda_home}/lib64", "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, PKG / "build" / "torch_ops.log")
    stamp_file.write_text(stamp)
    return TORCH_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_torch_shim(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB, TORCH_LIB)
