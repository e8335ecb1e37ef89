"""In-tree build of the native libraries (sm_100a only).

  lib/libsk_w2a8.so        CUDA kernels + C ABI (include/sk_w2a8.h), built with nvcc, no torch dependency
  lib/libsk_w2a8_torch.so  PyTorch C++ extension that marshals tensors into the C ABI

Both are rebuilt only when a source is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
_CSRC = os.path.join(_PKG, "csrc")
LIB_DIR = os.path.join(_PKG, "lib")
CUDA_LIB = os.path.join(LIB_DIR, "libsk_w2a8.so")
TORCH_LIB = os.path.join(LIB_DIR, "libsk_w2a8_torch.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose and proc.stderr.strip():
        print(proc.stderr, file=sys.stderr)


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def build_cuda_lib(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    srcs = [os.path.join(_CSRC, f) for f in ("sk_w2a8.cu", "w2a8_umma.cuh", "ptx_sm100.cuh")]
    srcs.append(os.path.join(_ROOT, "include", "sk_w2a8.h"))
    extra = [os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith((".cuh", ".cu", ".h"))]
    if force or _newer(CUDA_LIB, set(srcs + extra)):
        os.makedirs(LIB_DIR, exist_ok=True)
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
              ["-o", CUDA_LIB, os.path.join(_CSRC, "sk_w2a8.cu")]
        _run(cmd, verbose)
    return CUDA_LIB


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(_CSRC, "torch_ext.cpp")
    build_cuda_lib(force=False, verbose=verbose)
    if force or _newer(TORCH_LIB, [src, os.path.join(_ROOT, "include", "sk_w2a8.h")]):
        import torch
        from torch.utils import cpp_extension as ce
        incs = [f"-I{p}" for p in ce.include_paths("cuda")]
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
               "-DTORCH_API_INCLUDE_EXTENSION_H", "-Wno-deprecated-declarations"] + incs + \
              ["-o", TORCH_LIB, src, f"-L{LIB_DIR}", "-lsk_w2a8", f"-L{tlib}", "-lc10", "-lc10_cuda",
               "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-L/usr/local/cuda/lib64", "-lcudart",
               "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
        _run(cmd, verbose)
    return TORCH_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda_lib(force, verbose)
    build_torch_ext(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
