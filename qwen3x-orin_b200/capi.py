"""ctypes binding of include/q3x_b200.h.  Every wrapper takes raw device addresses (ints) or objects
with a ``data_ptr()`` method (torch tensors) and returns the entry point's int status unchanged;
``check`` turns a non-zero status into an exception."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# the in-tree build, unless Q3X_B200_LIBRARY names another build of the same library
LIB_PATH = os.environ.get("Q3X_B200_LIBRARY") or os.path.join(_PKG, "libq3x_b200.so")
HOST_LIB_PATH = os.path.join(_PKG, "libq3x_b200_host.so")

CUDA_SUCCESS = 0
CUDA_ERROR_INVALID_VALUE = 1
CUDA_ERROR_NOT_SUPPORTED = 801

_p = C.c_void_p
_z = C.c_size_t
_f = C.c_float
_i = C.c_int

# name -> (restype, argtypes); the order of every argument list is the header's
SIGNATURES = {
    "q3x_b200_abi_version": (_i, []),
    "q3x_b200_error_string": (C.c_char_p, [_i]),
    "q3x_b200_embedding_gather": (_i, [_p, _z, _z, _p, _z, _p, _p]),
    "q3x_b200_embedding_gather_one": (_i, [_p, _z, _z, _z, _p, _p]),
    "q3x_b200_rms_norm": (_i, [_p, _p, _z, _z, _f, _i, _p, _p]),
    "q3x_b200_rms_norm_silu_gate": (_i, [_p, _p, _p, _z, _z, _f, _p, _p]),
    "q3x_b200_l2_normalize_heads": (_i, [_p, _z, _z, _f, _f, _p, _p]),
    "q3x_b200_residual_add": (_i, [_p, _p, _z, _p, _p]),
    "q3x_b200_residual_add_rms_norm": (_i, [_p, _p, _p, _z, _z, _f, _p, _p, _p]),
    "q3x_b200_nvfp4_group_count": (_z, [_z, _z]),
    "q3x_b200_nvfp4_scratch_words": (_z, [_z, _z]),
    "q3x_b200_group_amax": (_i, [_p, _z, _z, _z, _p, _p]),
    "q3x_b200_amax_to_global_scale": (_i, [_p, _z, _p, _p]),
    "q3x_b200_nvfp4_quantize": (_i, [_p, _z, _z, _z, _p, _p, _p, _p]),
    "q3x_b200_nvfp4_quantize_dynamic": (_i, [_p, _z, _z, _z, _p, _p, _p, _p, _p]),
    "q3x_b200_nvfp4_swizzled_scale_bytes": (_z, [_z, _z]),
    "q3x_b200_nvfp4_swizzle_block_scales": (_i, [_p, _z, _z, _p, _p]),
    "q3x_b200_bf16_gemm_workspace_bytes": (_z, [_z, _z, _z]),
    "q3x_b200_bf16_gemm_bf16": (_i, [_p, _p, _z, _z, _z, _p, _p, _z, _p]),
    "q3x_b200_bf16_gemm_scaled_bf16": (_i, [_p, _f, _p, _z, _z, _z, _p, _p, _z, _p]),
    "q3x_b200_fp8_weights_to_bf16": (_i, [_p, _z, _p, _p]),
    "q3x_b200_nvfp4_weights_to_bf16": (_i, [_p, _p, _z, _z, _p, _p]),
    "q3x_b200_fp8_gemm_workspace_bytes": (_z, [_z, _z, _z]),
    "q3x_b200_fp8_gemm_bf16": (_i, [_p, _f, _p, _z, _z, _z, _p, _p, _z, _p]),
    "q3x_b200_nvfp4_transpose_block_scales": (_i, [_p, _z, _z, _p, _p]),
    "q3x_b200_nvfp4_w4a16_gemm_workspace_bytes": (_z, [_z, _z, _z]),
    "q3x_b200_nvfp4_w4a16_gemm_bf16": (_i, [_p, _p, _f, _p, _z, _z, _z, _p, _p, _z, _p]),
    "q3x_b200_nvfp4_gemm_workspace_bytes": (_z, [_z, _z, _z, _z]),
    "q3x_b200_nvfp4_gemm_bf16": (_i, [_p, _p, _p, _z, _p, _p, _f, _z, _z, _z, _p, _p, _z, _p]),
    "q3x_b200_residual_add_rms_norm_nvfp4": (_i, [_p, _p, _p, _z, _z, _f, _z, _p, _p, _p, _p, _p, _p, _p]),
    "q3x_b200_rms_norm_silu_gate_nvfp4": (_i, [_p, _p, _p, _z, _z, _z, _f, _z, _p, _p, _p, _p, _p, _p]),
    "q3x_b200_residual_add_rms_norm_nvfp4_single_pass": (_i, [_p, _p, _p, _z, _z, _f, _z, _p, _p, _p, _p, _p, _p, _p]),
    "q3x_b200_silu_mul_nvfp4": (_i, [_p, _p, _z, _z, _z, _p, _p, _p, _p, _p, _p]),
    "q3x_b200_sigmoid_gate_nvfp4": (_i, [_p, _p, _z, _z, _z, _p, _p, _p, _p, _p, _p]),
    "q3x_b200_rms_norm_silu_gate_nvfp4_single_pass": (_i, [_p, _p, _p, _z, _z, _z, _f, _z, _p, _p, _p, _p, _p, _p]),
    "q3x_b200_static_scratch_max_tokens": (_z, []),
    "q3x_b200_residual_add_rms_norm_nvfp4_static_scratch": (_i, [_p, _p, _p, _z, _z, _f, _z, _p, _p, _p, _p, _p, _p]),
    "q3x_b200_debug_encode": (_i, [_p, _z, _i, _p, _p]),
    "q3x_b200_debug_intermediate": (_i, [_p, _z, _i, _f, _f, _p, _p]),
    "q3x_b200_debug_stale_error": (_i, [_i]),
    "q3x_b200_split_interleaved_q_gate": (_i, [_p, _z, _z, _p, _p, _p]),
    "q3x_b200_partial_neox_rope_256_64": (_i, [_p, _p, _p, _z, _p, _p]),
    "q3x_b200_qk_partial_neox_rope": (_i, [_p, _p, _p, _p, _z, _z, _p]),
    "q3x_b200_full_attention_preprocess": (_i, [_p, _p, _p, _p, _f, _p, _p, _p, _p, _z, _z, _p]),
    "q3x_b200_sigmoid_gate": (_i, [_p, _p, _z, _p, _p]),
    "q3x_b200_silu_mul": (_i, [_p, _p, _z, _p, _p]),
    "q3x_b200_silu_mul_merged": (_i, [_p, _z, _z, _p, _p]),
    "q3x_b200_fp32_to_bf16": (_i, [_p, _z, _p, _p]),
    "q3x_b200_causal_conv1d_silu": (_i, [_p, _z, _z, _p, _p, _p, _p]),
    "q3x_b200_causal_conv1d_silu_l2norm": (_i, [_p, _z, _p, _p, _f, _f, _p, _p]),
    "q3x_b200_causal_conv1d_silu_compact_qk": (_i, [_p, _z, _p, _p, _p, _f, _f, _p, _p, _p]),
    "q3x_b200_bf16_gemv": (_i, [_p, _p, _z, _z, _p, _p, _p]),
    "q3x_b200_fp8_gemv": (_i, [_p, _f, _p, _z, _z, _p, _p, _p]),
    "q3x_b200_nvfp4_gemv": (_i, [_p, _p, _f, _p, _z, _z, _p, _p, _p]),
    "q3x_b200_gated_delta_net_update": (_i, [_p, _z, _p, _p, _p, _p, _p, _p, _f, _p, _p]),
    "q3x_b200_gated_delta_net_chunked_workspace_bytes": (_z, [_z]),
    "q3x_b200_gated_delta_net_chunked_select_path": (_i, [_i]),
    "q3x_b200_gated_delta_net_update_chunked": (_i, [_p, _z, _p, _p, _p, _p, _p, _p, _f, _p, _p, _z, _p]),
    "q3x_b200_gated_delta_net_update_rms_norm_silu_gate": (_i, [_p, _z, _p, _p, _p, _p, _p, _p, _f, _p, _p, _f, _p, _p]),
    "q3x_b200_gqa_decode_workspace_floats": (_z, [_z]),
    "q3x_b200_gqa_attention_decode_sigmoid_gate": (_i, [_p, _p, _p, _z, _f, _p, _z, _p, _p, _p]),
    "q3x_b200_gqa_attention_prefill_sigmoid_gate": (_i, [_p, _p, _p, _p, _z, _z, _f, _p, _p]),
    "q3x_b200_gqa_prefill_select_path": (_i, [_i]),
    "q3x_b200_gqa_prefill_tcgen05_error": (_i, []),
    "q3x_b200_softmax": (_i, [_p, _z, _z, _p, _p]),
    "q3x_b200_bf16_greedy_argmax": (_i, [_p, _z, _p, _p]),
}

_lib = None


class Q3xError(RuntimeError):
    def __init__(self, name, status):
        self.status = status
        msg = lib().q3x_b200_error_string(status)
        super().__init__(f"{name} returned {status} ({msg.decode() if msg else '?'})")


def load(path: str = LIB_PATH):
    """dlopen the CUDA library and declare every entry point.  Raises when the library is missing:
    the operators have no other implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python qwen3x-orin_b200/build.py` "
                "(the operators are CUDA-only, there is no fallback)")
        handle = C.CDLL(path, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError = the library does not export the symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def lib():
    return load()


def ptr(x):
    """Device address of a tensor-like, or the int / None given."""
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    return int(x)


def call(name: str, *args) -> int:
    """Calls an entry point; tensor-likes are replaced by their device address."""
    fn = getattr(lib(), name)
    return fn(*[ptr(a) if (hasattr(a, "data_ptr") or a is None) else a for a in args])


def check(name: str, *args) -> None:
    st = call(name, *args)
    if st != CUDA_SUCCESS:
        raise Q3xError(name, st)
