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

OBJ = os.path.join(PKG, "_build")
CUDA_SOURCES = ["pointwise.cu", "row_norms.cu", "attention_preprocess.cu", "gdn_conv.cu", "embedding.cu", "nvfp4.cu",
                "fused_nvfp4.cu", "gdn_recurrence.cu", "gdn_chunked.cu", "gqa_decode.cu", "gqa_prefill.cu", "logits_ops.cu", "gemv.cu", "nvfp4_gemm.cu", "fp8_gemm.cu", "nvfp4_w4a16_gemm.cu", "bf16_gemm.cu"]
# sources instantiated from the CUTLASS / CuTe header tree (found inside an installed Python package, see _cutlass)
CUTLASS_SOURCES = {"nvfp4_gemm.cu", "fp8_gemm.cu", "nvfp4_w4a16_gemm.cu", "bf16_gemm.cu"}
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


def _cutlass() -> str:
    """Root of a CUTLASS tree (include/ and tools/util/include/) with the sm100 block-scaled collectives:
    Q3X_B200_CUTLASS, else the tree vendored inside the flashinfer package."""
    import importlib.util

    candidates = [os.environ.get("Q3X_B200_CUTLASS")]
    spec = importlib.util.find_spec("flashinfer")
    if spec is not None and spec.submodule_search_locations:
        candidates.append(os.path.join(list(spec.submodule_search_locations)[0], "data", "cutlass"))
    for root in candidates:
        if root and os.path.exists(os.path.join(root, "include", "cutlass", "gemm", "collective", "builders",
                                                "sm100_blockscaled_umma_builder.inl")):
            return root
    raise RuntimeError("no CUTLASS tree with the sm100 block-scaled builders found (set Q3X_B200_CUTLASS)")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    sources = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = sources + [os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith((".cuh", ".hpp"))]
    deps.append(os.path.join(ROOT, "include", "q3x_b200.h"))
    headers = deps[len(sources):]
    os.makedirs(OBJ, exist_ok=True)
    objects, jobs = [], []
    for name, src in zip(CUDA_SOURCES, sources):
        obj = os.path.join(OBJ, name[:-3] + ".o")
        objects.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", src, "-o", obj]
            if name in CUTLASS_SOURCES:
                root = _cutlass()
                cmd[1:1] = ["--expt-relaxed-constexpr", "-diag-suppress", "20012", "-I", os.path.join(root, "include"),
                            "-I", os.path.join(root, "tools", "util", "include")]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(subprocess.Popen(cmd))
    failed = [j.args for j in jobs if j.wait() != 0]
    if failed:
        raise RuntimeError(f"nvcc failed: {failed[0]}")
    if force or jobs or _stale(LIB, objects):
        subprocess.run([_nvcc(), *NVCC_FLAGS, "-shared", "-o", LIB, *objects], check=True)
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
