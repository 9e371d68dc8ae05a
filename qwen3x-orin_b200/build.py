"""Builds libq3x_b200.so (CUDA kernels + C ABI, sm_100a) and libq3x_b200_host.so (the C++17 mirror of
the reference operator API) in-tree with nvcc / g++.  nvcc cross-compiles without a GPU."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
LIB = os.path.join(PKG, "libq3x_b200.so")
HOST_LIB = os.path.join(PKG, "libq3x_b200_host.so")

CUDA_SOURCES = ["pointwise.cu", "row_norms.cu", "attention_preprocess.cu", "gdn_conv.cu", "embedding.cu", "nvfp4.cu",
                "fused_nvfp4.cu", "gdn_recurrence.cu", "gqa_decode.cu", "logits_ops.cu", "gemv.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    # IEEE arithmetic everywhere: no fast-math, accurate division / sqrt, denormals kept
    "--ftz=false", "--prec-div=true", "--prec-sqrt=true",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    sources = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = sources + [os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith((".cuh", ".hpp"))]
    deps.append(os.path.join(ROOT, "include", "q3x_b200.h"))
    if force or _stale(LIB, deps):
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-shared", "-o", LIB, *sources]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.run(cmd, check=True)
    return LIB


def build_host(force: bool = False) -> str | None:
    if not os.path.isdir(HOST):
        return None
    sources = [os.path.join(HOST, s) for s in sorted(os.listdir(HOST)) if s.endswith(".cpp")]
    if not sources:
        return None
    deps = sources + [os.path.join(HOST, h) for h in os.listdir(HOST) if h.endswith((".hpp", ".h"))]
    deps.append(os.path.join(ROOT, "include", "q3x_b200.h"))
    if force or _stale(HOST_LIB, deps + [LIB]):
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"),
               "-I", HOST, "-o", HOST_LIB, *sources, "-L", PKG, "-lq3x_b200", "-Wl,-rpath,$ORIGIN"]
        subprocess.run(cmd, check=True)
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", LIB)
