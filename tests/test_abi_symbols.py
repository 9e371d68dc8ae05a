"""CPU-side checks of the drop-in boundary: the C-ABI library builds for sm_100a, loads without a
GPU, exports every symbol include/q3x_b200.h declares, and rejects bad arguments on the host
before any device work (those paths never touch the GPU, so they run here too)."""
import ctypes as C
import importlib
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def capi():
    pkg = importlib.import_module("qwen3x-orin_b200")
    build = importlib.import_module("qwen3x-orin_b200.build")
    build.build_all()
    pkg.capi.load()
    return pkg.capi


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "q3x_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q3x_b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(capi):
    names = declared_symbols()
    assert len(names) >= 25
    handle = C.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/q3x_b200.h but not exported"
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == names, "capi binds a symbol the header does not declare"
    assert capi.lib().q3x_b200_abi_version() == 1


def test_no_cpu_fallback_when_library_is_missing(tmp_path):
    pkg = importlib.import_module("qwen3x-orin_b200")
    saved = pkg.capi._lib
    pkg.capi._lib = None
    try:
        with pytest.raises(RuntimeError, match="no fallback"):
            pkg.capi.load(str(tmp_path / "libq3x_b200.so"))
    finally:
        pkg.capi._lib = saved


def test_product_sources_never_reference_the_oracle():
    """The oracle is test infrastructure: nothing under the package may import, link or call it."""
    pkg_dir = os.path.join(ROOT, "qwen3x-orin_b200")
    for base, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".cpp", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


INVALID, OK = 1, 0
A = 0x10000  # a fake, never dereferenced device address: these calls must fail before any launch


def test_host_side_argument_checks(capi):
    c = capi.call
    nan = float("nan")
    # epsilon must be finite and positive (src/kernels/reference/decode_ops.cu:155-157)
    assert c("q3x_b200_rms_norm", A, A + 0x1000, 1, 8, 0.0, 1, A + 0x2000, None) == INVALID
    assert c("q3x_b200_rms_norm", A, A + 0x1000, 1, 8, nan, 1, A + 0x2000, None) == INVALID
    assert c("q3x_b200_rms_norm", A, A + 0x1000, 1, 8, -1e-6, 1, A + 0x2000, None) == INVALID
    # null pointers on a non-empty shape
    assert c("q3x_b200_rms_norm", None, A, 1, 8, 1e-6, 1, A + 0x1000, None) == INVALID
    assert c("q3x_b200_residual_add", A, None, 8, A + 0x1000, None) == INVALID
    assert c("q3x_b200_silu_mul", A, A, 8, None, None) == INVALID
    # empty shapes succeed even with null pointers
    assert c("q3x_b200_rms_norm", None, None, 0, 8, 1e-6, 1, None, None) == OK
    assert c("q3x_b200_residual_add", None, None, 0, None, None) == OK
    assert c("q3x_b200_embedding_gather", None, 10, 0, None, 5, None, None) == OK
    assert c("q3x_b200_full_attention_preprocess", None, None, None, None, 1e-6, None, None, None, None, 0, 0, None) == OK
    assert c("q3x_b200_causal_conv1d_silu", None, 0, 10240, None, None, None, None) == OK
    assert c("q3x_b200_nvfp4_quantize", None, 0, 64, 0, None, None, None, None) == OK
    # size overflow
    big = (1 << 63)
    assert c("q3x_b200_rms_norm", A, A, big, 4, 1e-6, 1, A, None) == INVALID
    assert c("q3x_b200_l2_normalize_heads", A, big, 4, 1e-6, 1.0, A, None) == INVALID
    assert c("q3x_b200_residual_add", A, A + big, big, A, None) == INVALID
    # residual add: inputs must be disjoint, partial output overlap is rejected, exact alias is not
    assert c("q3x_b200_residual_add", A, A + 8, 64, A + 0x1000, None) == INVALID
    assert c("q3x_b200_residual_add", A, A + 0x1000, 64, A + 2, None) == INVALID
    # fused residual + norm: residual_out overlapping anything, normalized partially overlapping right
    H = 5120 * 2
    assert c("q3x_b200_residual_add_rms_norm", A, A + H, A + 2 * H, 1, 5120, 1e-6, A, A + 3 * H, None) == INVALID
    assert c("q3x_b200_residual_add_rms_norm", A, A + H, A + 2 * H, 1, 5120, 1e-6, A + 3 * H, A + H + 2, None) == INVALID
    assert c("q3x_b200_residual_add_rms_norm", A, A + H, A + 2 * H, 1, 5120, 1e-6, A + 3 * H, A, None) == INVALID
    # preprocess: writable tensors must not overlap inputs or each other
    q = 24 * 256 * 2
    args = dict(qg=A, key=A + 0x100000, qw=A + 0x200000, kw=A + 0x201000, qo=A + 0x300000, go=A + 0x400000,
                cos=A + 0x500000, sin=A + 0x600000)
    def pre(**kw):
        a = {**args, **kw}
        return c("q3x_b200_full_attention_preprocess", a["qg"], a["key"], a["qw"], a["kw"], 1e-6, a["qo"], a["go"],
                 a["cos"], a["sin"], 0, 1, None)
    assert pre(qo=A + 2) == INVALID and pre(go=args["qo"] + q - 2) == INVALID and pre(key=args["cos"]) == INVALID
    assert pre(qo=None) == INVALID
    # split: three pairwise overlaps (src/kernels/reference/layout_ops.cu:77-86)
    assert c("q3x_b200_split_interleaved_q_gate", A, 4, 8, A + 16, A + 0x1000, None) == INVALID
    assert c("q3x_b200_split_interleaved_q_gate", A, 4, 8, A + 0x1000, A + 0x1000 + 8, None) == INVALID
    # conv: geometry and exact aliases (src/runtime/reference/gdn_decode.cpp:80-88)
    C_ = 10240
    assert c("q3x_b200_causal_conv1d_silu", A, 1, 64, A + 0x100000, A + 0x200000, A + 0x300000, None) == INVALID
    assert c("q3x_b200_causal_conv1d_silu", A, 1, C_, A, A + 0x200000, A + 0x300000, None) == INVALID
    assert c("q3x_b200_causal_conv1d_silu", A, 1, C_, A + 0x100000, A + 0x200000, A + 0x200000, None) == INVALID
    assert c("q3x_b200_causal_conv1d_silu_l2norm", A, 1, A + 0x100000, A + 0x200000, 1e-6, 1.0, A, None) == INVALID
    # embedding: vocabulary of zero, overlapping table / ids / output
    assert c("q3x_b200_embedding_gather", A, 0, 8, A + 0x1000, 1, A + 0x2000, None) == INVALID
    assert c("q3x_b200_embedding_gather", A, 16, 8, A + 8, 1, A + 0x2000, None) == INVALID
    # NVFP4: columns must be a multiple of 16
    assert c("q3x_b200_nvfp4_quantize", A, 1, 24, 0, A + 0x1000, A + 0x2000, A + 0x3000, None) == INVALID
    assert c("q3x_b200_nvfp4_quantize_dynamic", A, 1, 32, 0, None, A + 0x1000, A + 0x2000, A + 0x3000, None) == INVALID
    assert capi.lib().q3x_b200_nvfp4_group_count(513, 512) == 2
    assert capi.lib().q3x_b200_nvfp4_group_count(513, 0) == 1
    assert capi.lib().q3x_b200_nvfp4_group_count(0, 512) == 0


def test_host_side_argument_checks_of_the_tensor_core_entries(capi):
    """The panel projections, the chunked recurrence and the path switches: everything these refuse they refuse on the
    host, before any CUDA call (so this runs without a GPU)."""
    c, L = capi.call, capi.lib()
    B = A + (1 << 30)
    # dense scaled projection and the exact widenings that feed it
    assert c("q3x_b200_bf16_gemm_scaled_bf16", A, float("nan"), B, 64, 64, 128, B + (1 << 24), None, 0, None) == INVALID
    assert c("q3x_b200_bf16_gemm_scaled_bf16", A, 1.0, B, 64, 60, 128, B + (1 << 24), None, 0, None) == INVALID   # N % 8
    assert c("q3x_b200_bf16_gemm_scaled_bf16", A, 1.0, B, 64, 64, 100, B + (1 << 24), None, 0, None) == INVALID   # K % 8
    assert c("q3x_b200_bf16_gemm_scaled_bf16", A, 1.0, B, 64, 64, 128, A + 64, None, 0, None) == INVALID          # out on W
    assert c("q3x_b200_bf16_gemm_scaled_bf16", None, 1.0, B, 64, 64, 128, B + (1 << 24), None, 0, None) == INVALID
    assert c("q3x_b200_bf16_gemm_scaled_bf16", A, 1.0, B, 0, 64, 128, B + (1 << 24), None, 0, None) == OK
    assert c("q3x_b200_fp8_weights_to_bf16", A, 24, B, None) == INVALID            # whole 16-element vectors only
    assert c("q3x_b200_fp8_weights_to_bf16", A, 64, A + 32, None) == INVALID        # overlap
    assert c("q3x_b200_fp8_weights_to_bf16", None, 64, B, None) == INVALID
    assert c("q3x_b200_fp8_weights_to_bf16", A, 0, B, None) == OK
    assert c("q3x_b200_nvfp4_weights_to_bf16", A, B, 8, 24, B + (1 << 24), None) == INVALID    # cols % 16
    assert c("q3x_b200_nvfp4_weights_to_bf16", A, B, 8, 32, A + 64, None) == INVALID           # out on the codes
    assert c("q3x_b200_nvfp4_weights_to_bf16", A, None, 8, 32, B + (1 << 24), None) == INVALID
    assert c("q3x_b200_nvfp4_weights_to_bf16", A, B, 0, 32, B + (1 << 24), None) == OK
    # chunked recurrence: workspace arithmetic and refusals
    one = L.q3x_b200_gated_delta_net_chunked_workspace_bytes(64)
    assert one > 0 and L.q3x_b200_gated_delta_net_chunked_workspace_bytes(1) == one
    assert L.q3x_b200_gated_delta_net_chunked_workspace_bytes(65) == 2 * (one - 256) + 256
    assert L.q3x_b200_gated_delta_net_chunked_workspace_bytes(0) == 0
    state, ws = A + (1 << 26), B + (1 << 28)
    chunked = lambda **kw: c("q3x_b200_gated_delta_net_update_chunked", A, kw.get("tokens", 64), A + (1 << 22), A + (1 << 23),
                             A + (1 << 24), A + (1 << 24) + 4096, state, kw.get("state_out", state), kw.get("eps", 1e-6),
                             kw.get("out", B), kw.get("ws", ws), kw.get("ws_bytes", one), None)
    assert chunked(ws_bytes=one - 16) == INVALID
    assert chunked(ws=None) == INVALID
    assert chunked(eps=0.0) == INVALID
    assert chunked(out=state) == INVALID
    assert chunked(state_out=state + 64) == INVALID   # partial overlap of the two states
    assert chunked(ws=B) == INVALID                   # workspace on the output
    assert chunked(tokens=0) == OK
    # path switches take 0 or 1
    for name in ("q3x_b200_gated_delta_net_chunked_select_path", "q3x_b200_gqa_prefill_select_path"):
        assert c(name, 2) == INVALID and c(name, -1) == INVALID
    assert c("q3x_b200_gated_delta_net_chunked_select_path", 0) == OK and c("q3x_b200_gqa_prefill_select_path", 1) == OK
