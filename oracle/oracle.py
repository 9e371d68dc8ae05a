"""numpy/ctypes front end of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two libraries sit behind this module:

* ``libq3x_oracle.so`` -- the plain-C restatement of the reference's host reference ops
  (``q3x_oracle.c``); always available after ``make -C oracle oracle``.
* ``_ref/libq3x_ref.so`` -- the reference project's own sources compiled from a reference
  checkout (``make -C oracle ref``); present only where a checkout was available at build time.

Only the tests, the smoke check and the bench's CPU-baseline leg import this module.  The CUDA
product path never does: it has no CPU fallback.

bf16 tensors are numpy ``uint16`` arrays holding raw bfloat16 bits.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libq3x_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libq3x_ref.so")

STATUS_OK = 0
STATUS_INVALID_ARGUMENT = 1
STATUS_INVALID_DIMENSION = 2
STATUS_SIZE_OVERFLOW = 3
STATUS_TOKEN_OUT_OF_RANGE = 4
STATUS_INVALID_ALIAS = 5
STATUS_INVALID_COLUMN_COUNT = 6

_u16p = C.POINTER(C.c_uint16)
_u8p = C.POINTER(C.c_uint8)
_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)
_sz = C.c_size_t


def reference_dir() -> str:
    """Where a checkout of the reference project is looked for: ``$Q3X_REFERENCE_DIR``, else the
    directory ``reference`` beside this repository (the Makefile's default)."""
    return os.environ.get("Q3X_REFERENCE_DIR") or os.path.abspath(os.path.join(_HERE, "..", "..", "reference"))


def build(force: bool = False) -> None:
    """Compile the restatement (and, where a reference checkout exists, ``_ref``)."""
    sources = [os.path.join(_HERE, n) for n in ("q3x_oracle.c", "q3x_oracle_core.c", "q3x_oracle.h")]
    if force or not os.path.exists(_ORACLE_SO) or os.path.getmtime(_ORACLE_SO) < max(map(os.path.getmtime, sources)):
        subprocess.run(["make", "-C", _HERE, "oracle"], check=True, capture_output=True)
    shim = os.path.join(_HERE, "ref_shim.cpp")
    if os.path.isdir(os.path.join(reference_dir(), "src", "runtime", "reference")) and (
            force or not os.path.exists(_REF_SO) or os.path.getmtime(_REF_SO) < os.path.getmtime(shim)):
        subprocess.run(["make", "-C", _HERE, "ref", f"REFERENCE={reference_dir()}"], check=True, capture_output=True)


def _p(a, ty):
    if a is None:
        return None
    return a.ctypes.data_as(ty)


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16, a.dtype
    return a


class _Lib:
    def __init__(self, path):
        self.lib = C.CDLL(path)

    def fn(self, name, restype, *argtypes):
        f = getattr(self.lib, name)
        f.restype = restype
        f.argtypes = list(argtypes)
        return f


_oracle = None
_ref = None


def oracle_lib():
    global _oracle
    if _oracle is None:
        if not os.path.exists(_ORACLE_SO):
            build()
        L = _Lib(_ORACLE_SO)
        i = C.c_int
        f = C.c_float
        L.decode_bf16 = L.fn("q3x_oracle_decode_bf16", f, C.c_uint16)
        L.encode_bf16 = L.fn("q3x_oracle_encode_bf16", C.c_uint16, f)
        L.fp32_to_bf16 = L.fn("q3x_oracle_fp32_to_bf16", i, _f32p, _sz, _u16p)
        L.embedding = L.fn("q3x_oracle_embedding_gather", i, _u16p, _sz, _sz, _u32p, _sz, _u16p)
        L.rms_norm = L.fn("q3x_oracle_rms_norm", i, _u16p, _u16p, _sz, f, i, _u16p)
        L.headwise = L.fn("q3x_oracle_headwise_rms_norm", i, _u16p, _u16p, _u16p, _sz, _sz, f, i, _u16p)
        L.residual_add = L.fn("q3x_oracle_residual_add", i, _u16p, _u16p, _sz, _u16p)
        L.residual_norm = L.fn("q3x_oracle_residual_add_rms_norm", i, _u16p, _u16p, _u16p, _sz, _sz, f,
                               _u16p, _u16p)
        L.silu_mul = L.fn("q3x_oracle_silu_mul", i, _u16p, _u16p, _sz, _u16p)
        L.silu_mul_merged = L.fn("q3x_oracle_silu_mul_merged", i, _u16p, _sz, _sz, _u16p)
        L.sigmoid_gate = L.fn("q3x_oracle_sigmoid_gate", i, _u16p, _u16p, _sz, _u16p)
        L.l2 = L.fn("q3x_oracle_l2_normalize_heads", i, _u16p, _sz, _sz, f, f, _u16p)
        L.rope = L.fn("q3x_oracle_partial_neox_rope_256_64", i, _u16p, _f32p, _f32p, _sz, _u16p)
        L.rope_tables = L.fn("q3x_oracle_rope_tables", None, _sz, _sz, _f32p, _f32p)
        L.split = L.fn("q3x_oracle_split_interleaved_q_gate", i, _u16p, _sz, _sz, _u16p, _u16p)
        L.preprocess = L.fn("q3x_oracle_full_attention_preprocess", i, _u16p, _u16p, _u16p, _u16p, f,
                            _u16p, _u16p, _f32p, _f32p, _sz, _sz)
        L.conv = L.fn("q3x_oracle_causal_conv1d_silu", i, _u16p, _sz, _sz, _u16p, _u16p, _u16p)
        L.decode_e2m1 = L.fn("q3x_oracle_decode_e2m1", f, C.c_uint8)
        L.decode_e4m3 = L.fn("q3x_oracle_decode_e4m3fn", f, C.c_uint8)
        L.encode_e4m3 = L.fn("q3x_oracle_encode_e4m3fn", C.c_uint8, f)
        L.encode_e2m1 = L.fn("q3x_oracle_encode_e2m1", C.c_uint8, f)
        L.dequant = L.fn("q3x_oracle_nvfp4_dequantize", i, _u8p, _u8p, f, _sz, _sz, _f32p)
        L.quant = L.fn("q3x_oracle_nvfp4_quantize", i, _u16p, _sz, _sz, _sz, _u8p, _u8p, _f32p)
        L.quant_ws = L.fn("q3x_oracle_nvfp4_quantize_with_scales", i, _u16p, _sz, _sz, _sz, _f32p, _u8p,
                          _u8p)
        L.group_amax = L.fn("q3x_oracle_group_amax", i, _u16p, _sz, _sz, _sz, _f32p)
        L.gdn_update = L.fn("q3x_oracle_gated_delta_net_update", i, _u16p, _sz, _u16p, _u16p, _u16p, _u16p, _u16p,
                            _u16p, f, _u16p)
        L.softmax = L.fn("q3x_oracle_softmax", i, _f32p, _sz, _sz, _f32p)
        L.gqa = L.fn("q3x_oracle_gqa_attention", i, _u16p, _u16p, _u16p, _sz, _sz, _sz, _sz, f, _f32p, _u16p)
        L.gqa_gate = L.fn("q3x_oracle_gqa_attention_sigmoid_gate", i, _u16p, _u16p, _u16p, _sz, _sz, _sz, _sz, f,
                          _f32p, _u16p, _u16p)
        L.argmax = L.fn("q3x_oracle_bf16_greedy_argmax", i, _u16p, _sz, _u32p, _u16p, _u16p)
        L.bf16_gemv = L.fn("q3x_oracle_bf16_gemv", i, _u16p, _u16p, _sz, _sz, _f32p)
        L.nvfp4_gemv = L.fn("q3x_oracle_nvfp4_gemv", i, _u8p, _u8p, f, _u16p, _sz, _sz, _f32p)
        _oracle = L
    return _oracle


def have_ref() -> bool:
    return os.path.exists(_REF_SO)


def ref_lib():
    """The reference's own host ops (None when ``_ref`` was never built)."""
    global _ref
    if _ref is None:
        if not have_ref():
            return None
        L = _Lib(_REF_SO)
        i = C.c_int
        f = C.c_float
        L.embedding = L.fn("ref_embedding_gather", i, _u16p, _sz, _sz, _sz, _u16p)
        L.centered = L.fn("ref_centered_rms_norm", i, _u16p, _u16p, _sz, f, _u16p)
        L.plain = L.fn("ref_plain_rms_norm", i, _u16p, _u16p, _sz, f, _u16p)
        L.head_centered = L.fn("ref_headwise_centered_rms_norm", i, _u16p, _u16p, _sz, _sz, f, _u16p)
        L.head_plain = L.fn("ref_headwise_plain_rms_norm", i, _u16p, _u16p, _sz, _sz, f, _u16p)
        L.head_plain_gate = L.fn("ref_headwise_plain_rms_norm_silu_gate", i, _u16p, _u16p, _u16p, _sz, _sz,
                                 f, _u16p)
        L.residual_add = L.fn("ref_residual_add", i, _u16p, _u16p, _sz, _u16p)
        L.fp32_to_bf16 = L.fn("ref_fp32_to_bf16", i, _f32p, _sz, _u16p)
        L.silu_mul = L.fn("ref_silu_mul", i, _u16p, _u16p, _sz, _u16p)
        L.sigmoid_gate = L.fn("ref_sigmoid_gate", i, _u16p, _u16p, _sz, _u16p)
        L.l2 = L.fn("ref_l2_normalize_heads", i, _u16p, _sz, _sz, f, _u16p)
        L.rope = L.fn("ref_partial_neox_rope_256_64", i, _u16p, _f32p, _f32p, _sz, _u16p)
        L.split = L.fn("ref_split_interleaved_q_gate", i, _u16p, _sz, _sz, _u16p, _u16p)
        L.conv = L.fn("ref_causal_conv1d_silu_update", i, _u16p, _u16p, _u16p, _u16p)
        L.decode_e2m1 = L.fn("ref_decode_e2m1", f, C.c_uint8)
        L.decode_e4m3 = L.fn("ref_decode_e4m3fn", f, C.c_uint8)
        L.unpack = L.fn("ref_unpack_e2m1_nibble", C.c_uint8, C.c_uint8, i)
        L.dequant = L.fn("ref_dequantize_nvfp4", i, _u8p, _u8p, f, _sz, _sz, _f32p)
        L.e4m3_value = L.fn("ref_e4m3_quantised_value", i, C.c_uint16, f, _f32p)
        L.gdn_update = L.fn("ref_gated_delta_net_update", i, _u16p, _u16p, _u16p, _u16p, _u16p, _u16p, _u16p, f, _u16p)
        L.softmax = L.fn("ref_softmax", i, _f32p, _sz, _sz, _f32p)
        L.gqa = L.fn("ref_gqa_attention", i, _u16p, _u16p, _u16p, _sz, _sz, _sz, _sz, f, _f32p, _sz, _u16p)
        L.bf16_gemv = L.fn("ref_bf16_gemv", i, _u16p, _u16p, _sz, _sz, _f32p)
        L.nvfp4_gemv = L.fn("ref_nvfp4_gemv", i, _u8p, _u8p, f, _u16p, _sz, _sz, _f32p)
        L.embedding_rows = L.fn("ref_embedding_gather_rows", i, _u16p, _sz, _sz, _u32p, _sz, _u16p)
        L.conv_rows = L.fn("ref_causal_conv1d_silu_update_rows", i, _u16p, _sz, _u16p, _u16p, _u16p)
        L.preprocess_rows = L.fn("ref_full_attention_preprocess_rows", i, _u16p, _u16p, _u16p, _u16p, f, _u16p,
                                 _u16p, _f32p, _f32p, _sz, _sz)
        _ref = L
    return _ref


# ------------------------------------------------------------------ bf16 helpers (numpy)

def bf16_decode(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bits -> float32 (exact)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_encode(values: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bits, the reference's rule (RNE, NaN quieted with payload kept):
    src/runtime/reference/decode_ops.cpp:22-33."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    u = v.view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + (0x7FFF + ((u >> 16) & 1))) >> 16
    quiet = (u >> 16) | 0x0040
    return np.where(nan, quiet, rounded).astype(np.uint16)


def bf16_is_nan(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16) & 0x7FFF) > 0x7F80


def bf16_ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in bf16 steps between two bit patterns (sign-magnitude mapped to a line).
    NaN vs NaN counts as 0, NaN vs number as a large distance."""
    a = np.asarray(a, dtype=np.uint16).astype(np.int32)
    b = np.asarray(b, dtype=np.uint16).astype(np.int32)

    def line(x):
        mag = x & 0x7FFF
        return np.where(x & 0x8000, -mag, mag)

    nan_a = (a & 0x7FFF) > 0x7F80
    nan_b = (b & 0x7FFF) > 0x7F80
    d = np.abs(line(a) - line(b))
    d = np.where(nan_a & nan_b, 0, d)
    d = np.where(nan_a ^ nan_b, 1 << 20, d)
    return d


# ------------------------------------------------------------------ restatement wrappers

def _check(st, allowed=(STATUS_OK,)):
    if st not in allowed:
        raise RuntimeError(f"oracle status {st}")
    return st


def embedding_gather(table, token_ids, out=None):
    L = oracle_lib()
    table = _u16(table)
    ids = np.ascontiguousarray(token_ids, dtype=np.uint32)
    vocab, hidden = table.shape
    if out is None:
        out = np.zeros((ids.size, hidden), dtype=np.uint16)
    st = L.embedding(_p(table, _u16p), vocab, hidden, _p(ids, _u32p), ids.size, _p(out, _u16p))
    _check(st, (STATUS_OK, STATUS_TOKEN_OUT_OF_RANGE))
    return out


def rms_norm_rows(x, weight, eps, centered=True, gate=None):
    """Row-wise RMSNorm over the last axis with one shared weight (headwise form)."""
    L = oracle_lib()
    x = _u16(x)
    weight = _u16(weight)
    dim = x.shape[-1]
    heads = x.size // dim if dim else 0
    out = np.empty_like(x)
    g = _u16(gate) if gate is not None else None
    _check(L.headwise(_p(x, _u16p), _p(weight, _u16p), _p(g, _u16p), heads, dim, eps, int(centered),
                      _p(out, _u16p)))
    return out


def residual_add(left, right):
    L = oracle_lib()
    left, right = _u16(left), _u16(right)
    out = np.empty_like(left)
    _check(L.residual_add(_p(left, _u16p), _p(right, _u16p), left.size, _p(out, _u16p)))
    return out


def residual_add_rms_norm(left, right, weight, eps):
    L = oracle_lib()
    left, right, weight = _u16(left), _u16(right), _u16(weight)
    tokens, hidden = left.shape
    res = np.empty_like(left)
    nrm = np.empty_like(left)
    _check(L.residual_norm(_p(left, _u16p), _p(right, _u16p), _p(weight, _u16p), tokens, hidden, eps,
                           _p(res, _u16p), _p(nrm, _u16p)))
    return res, nrm


def silu_mul(gate, up):
    L = oracle_lib()
    gate, up = _u16(gate), _u16(up)
    out = np.empty_like(gate)
    _check(L.silu_mul(_p(gate, _u16p), _p(up, _u16p), gate.size, _p(out, _u16p)))
    return out


def silu_mul_merged(merged):
    L = oracle_lib()
    merged = _u16(merged)
    tokens, two_i = merged.shape
    out = np.empty((tokens, two_i // 2), dtype=np.uint16)
    _check(L.silu_mul_merged(_p(merged, _u16p), tokens, two_i // 2, _p(out, _u16p)))
    return out


def sigmoid_gate(value, gate):
    L = oracle_lib()
    value, gate = _u16(value), _u16(gate)
    out = np.empty_like(value)
    _check(L.sigmoid_gate(_p(value, _u16p), _p(gate, _u16p), value.size, _p(out, _u16p)))
    return out


def l2_normalize_heads(x, eps, scale=1.0):
    L = oracle_lib()
    x = _u16(x)
    dim = x.shape[-1]
    out = np.empty_like(x)
    _check(L.l2(_p(x, _u16p), x.size // dim if dim else 0, dim, eps, scale, _p(out, _u16p)))
    return out


def rope_tables(first_position, positions):
    L = oracle_lib()
    cos = np.empty((positions, 32), dtype=np.float32)
    sin = np.empty((positions, 32), dtype=np.float32)
    L.rope_tables(first_position, positions, _p(cos, _f32p), _p(sin, _f32p))
    return cos, sin


def partial_rope(x, cos_row, sin_row):
    L = oracle_lib()
    x = _u16(x)
    cos_row = np.ascontiguousarray(cos_row, dtype=np.float32)
    sin_row = np.ascontiguousarray(sin_row, dtype=np.float32)
    out = np.empty_like(x)
    _check(L.rope(_p(x, _u16p), _p(cos_row, _f32p), _p(sin_row, _f32p), x.size // 256, _p(out, _u16p)))
    return out


def split_q_gate(x, heads, dim):
    L = oracle_lib()
    x = _u16(x)
    q = np.empty(heads * dim, dtype=np.uint16)
    g = np.empty(heads * dim, dtype=np.uint16)
    _check(L.split(_p(x, _u16p), heads, dim, _p(q, _u16p), _p(g, _u16p)))
    return q, g


def full_attention_preprocess(q_gate, key, q_w, k_w, eps, cos, sin, first_position):
    """Returns (q_out, gate_out, key_out); cos/sin are [positions,32] tables from position 0."""
    L = oracle_lib()
    q_gate = _u16(q_gate)
    key = _u16(key).copy()
    tokens = q_gate.shape[0]
    q = np.empty((tokens, 24, 256), dtype=np.uint16)
    g = np.empty((tokens, 24, 256), dtype=np.uint16)
    cos = np.ascontiguousarray(cos, dtype=np.float32)
    sin = np.ascontiguousarray(sin, dtype=np.float32)
    _check(L.preprocess(_p(q_gate, _u16p), _p(key, _u16p), _p(_u16(q_w), _u16p), _p(_u16(k_w), _u16p), eps,
                        _p(q, _u16p), _p(g, _u16p), _p(cos, _f32p), _p(sin, _f32p), first_position, tokens))
    return q, g, key


def causal_conv1d_silu(raw, weight, history):
    """Returns (out, new_history).  raw [T,C], weight [C,4], history [C,3]."""
    L = oracle_lib()
    raw, weight = _u16(raw), _u16(weight)
    hist = _u16(history).copy()
    tokens, channels = raw.shape
    out = np.empty_like(raw)
    _check(L.conv(_p(raw, _u16p), tokens, channels, _p(weight, _u16p), _p(hist, _u16p), _p(out, _u16p)))
    return out, hist


def nvfp4_quantize(x, rows_per_scale=0):
    """Returns (codes [R,C/2] u8, scales [R,C/16] u8, global_scales [groups] f32)."""
    L = oracle_lib()
    x = _u16(x)
    rows, cols = x.shape
    groups = 1 if rows_per_scale == 0 else (rows + rows_per_scale - 1) // rows_per_scale
    codes = np.empty((rows, cols // 2), dtype=np.uint8)
    scales = np.empty((rows, cols // 16), dtype=np.uint8)
    gs = np.empty(groups, dtype=np.float32)
    _check(L.quant(_p(x, _u16p), rows, cols, rows_per_scale, _p(codes, _u8p), _p(scales, _u8p), _p(gs, _f32p)))
    return codes, scales, gs


def nvfp4_quantize_with_scales(x, global_scales, rows_per_scale=0):
    L = oracle_lib()
    x = _u16(x)
    rows, cols = x.shape
    gs = np.ascontiguousarray(global_scales, dtype=np.float32)
    codes = np.empty((rows, cols // 2), dtype=np.uint8)
    scales = np.empty((rows, cols // 16), dtype=np.uint8)
    _check(L.quant_ws(_p(x, _u16p), rows, cols, rows_per_scale, _p(gs, _f32p), _p(codes, _u8p),
                      _p(scales, _u8p)))
    return codes, scales


def nvfp4_dequantize(codes, scales, global_scale):
    L = oracle_lib()
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, half = codes.shape
    out = np.empty((rows, half * 2), dtype=np.float32)
    _check(L.dequant(_p(codes, _u8p), _p(scales, _u8p), float(global_scale), rows, half * 2, _p(out, _f32p)))
    return out


def group_amax(x, rows_per_scale=0):
    L = oracle_lib()
    x = _u16(x)
    rows, cols = x.shape
    groups = 1 if rows_per_scale == 0 else (rows + rows_per_scale - 1) // rows_per_scale
    out = np.empty(groups, dtype=np.float32)
    _check(L.group_amax(_p(x, _u16p), rows, cols, rows_per_scale, _p(out, _f32p)))
    return out


# ------------------------------------------------------------------ operators between the fused layer ops

def gated_delta_net_update(conv_qkv, a, b, A_log, dt_bias, state, l2_eps):
    """Token-sequential GDN recurrence.  conv_qkv [T,10240], a / b [T,48], A_log / dt_bias [48],
    state [48,128,128].  Returns (out [T,6144], new_state)."""
    L = oracle_lib()
    conv_qkv, a, b = _u16(conv_qkv).reshape(-1, 10240), _u16(a).reshape(-1, 48), _u16(b).reshape(-1, 48)
    tokens = conv_qkv.shape[0]
    new_state = _u16(state).copy()
    out = np.empty((tokens, 6144), dtype=np.uint16)
    _check(L.gdn_update(_p(conv_qkv, _u16p), tokens, _p(a, _u16p), _p(b, _u16p), _p(_u16(A_log), _u16p),
                        _p(_u16(dt_bias), _u16p), _p(new_state, _u16p), _p(new_state, _u16p), l2_eps, _p(out, _u16p)))
    return out, new_state


def softmax(x):
    L = oracle_lib()
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    _check(L.softmax(_p(x, _f32p), x.shape[0], x.shape[1], _p(out, _f32p)))
    return out


def gqa_attention(q, k_cache, v_cache, scale, gate=None):
    """One query token [q_heads, dim] against caches [length, kv_heads, dim]; with `gate` the sigmoid output
    gate follows across a bf16 boundary.  Returns (out [q_heads, dim], probabilities [q_heads, length])."""
    L = oracle_lib()
    q, k_cache, v_cache = _u16(q), _u16(k_cache), _u16(v_cache)
    q_heads, dim = q.shape
    length, kv_heads, _ = k_cache.shape
    probs = np.empty((q_heads, length), dtype=np.float32)
    out = np.empty_like(q)
    if gate is None:
        _check(L.gqa(_p(q, _u16p), _p(k_cache, _u16p), _p(v_cache, _u16p), q_heads, kv_heads, length, dim, scale,
                     _p(probs, _f32p), _p(out, _u16p)))
    else:
        _check(L.gqa_gate(_p(q, _u16p), _p(k_cache, _u16p), _p(v_cache, _u16p), q_heads, kv_heads, length, dim, scale,
                          _p(probs, _f32p), _p(_u16(gate), _u16p), _p(out, _u16p)))
    return out, probs


def greedy_argmax(logits):
    """(index, value bits, has_nonfinite) of a bf16 vector."""
    L = oracle_lib()
    logits = _u16(logits).reshape(-1)
    idx, bits, bad = C.c_uint32(), C.c_uint16(), C.c_uint16()
    _check(L.argmax(_p(logits, _u16p), logits.size, C.byref(idx), C.byref(bits), C.byref(bad)))
    return idx.value, bits.value, bad.value


def bf16_gemv(w, x):
    L = oracle_lib()
    w, x = _u16(w), _u16(x)
    out = np.empty(w.shape[0], dtype=np.float32)
    _check(L.bf16_gemv(_p(w, _u16p), _p(x, _u16p), w.shape[0], w.shape[1], _p(out, _f32p)))
    return out


def nvfp4_gemv(packed, block_scales, weight_scale_2, x):
    L = oracle_lib()
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    block_scales = np.ascontiguousarray(block_scales, dtype=np.uint8)
    rows, cols = packed.shape[0], packed.shape[1] * 2
    out = np.empty(rows, dtype=np.float32)
    _check(L.nvfp4_gemv(_p(packed, _u8p), _p(block_scales, _u8p), float(weight_scale_2), _p(_u16(x), _u16p), rows, cols,
                        _p(out, _f32p)))
    return out


# ------------------------------------------------------------------ row-parallel driver

def parallel_rows(fn, row_count, threads):
    """Run ``fn(lo, hi)`` over contiguous row ranges on ``threads`` host threads (the C calls
    release the GIL).  Used by the CPU-baseline timing, where rows are independent."""
    threads = max(1, min(threads, row_count))
    bounds = [(row_count * i // threads, row_count * (i + 1) // threads) for i in range(threads)]
    with ThreadPoolExecutor(max_workers=threads) as pool:
        list(pool.map(lambda b: fn(*b), bounds))
