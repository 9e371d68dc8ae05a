"""GPU parity tests: every operator of libq3x_b200.so, called through the C ABI, against the CPU
oracle on the same seeded inputs.

Tolerances (the ones the path is specified with):
  * copies (embedding rows, q|gate split, RoPE pass-through dims) and the residual add: bit-exact;
  * every other bf16 output: within 1 bf16 ulp of the host reference op (NaN matches NaN);
  * NVFP4 codes, E4M3 block scales and FP32 global scales: bit-exact given the same bf16 operand.
Shapes replay those the reference's CUDA tests run (777-element vectors, 24x256 / 4x256 / 48x128
heads, 5x127 and 16x128 L2 heads, T in {1,2,7,8,31,32,...,511,512} tiles) plus sizes beyond them.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import fixtures as fx

pytestmark = pytest.mark.gpu

EPS = 1e-6


@pytest.fixture(scope="module")
def g():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    return gpu_util


def rng_for(*key):
    import zlib

    return np.random.default_rng([zlib.crc32(k.encode()) if isinstance(k, str) else int(k) for k in key])


# ----------------------------------------------------------------------------- pointwise

POINTWISE = [
    ("q3x_b200_residual_add", orc.residual_add, True),
    ("q3x_b200_silu_mul", orc.silu_mul, False),
    ("q3x_b200_sigmoid_gate", orc.sigmoid_gate, False),
]


@pytest.mark.parametrize("name,ref,exact", POINTWISE)
@pytest.mark.parametrize("count,misalign", [(17, 0), (777, 0), (777, 1), (8, 0), (100_003, 0), (1 << 20, 0), (4099, 3)])
def test_pointwise(g, name, ref, exact, count, misalign):
    rng = rng_for(count, misalign, 1)
    a = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (count,), 2.0), 0.01)
    b = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (count,), 2.0), 0.01)
    da, db = g.Dev(a, misalign), g.Dev(b, misalign)
    out = g.empty_like_dev((count,), fill=0x1234, misalign=misalign)
    g.capi.check(name, da, db, count, out, None)
    g.sync()
    want = ref(a, b)
    if exact:
        na = orc.bf16_is_nan(want)
        g.assert_bits_equal(out.get()[~na], want[~na], name)
        assert np.array_equal(orc.bf16_is_nan(out.get()), na)
    else:
        g.assert_bf16_within(out.get(), want, 1, 0.99, name)
    assert out.guards_intact() and np.array_equal(da.get(), a) and np.array_equal(db.get(), b)


@pytest.mark.parametrize("name,ref,exact", POINTWISE)
def test_pointwise_in_place(g, name, ref, exact):
    rng = rng_for(name, 2)
    a = fx.normal_bf16(rng, (5000,))
    b = fx.normal_bf16(rng, (5000,))
    for target in (0, 1):
        da, db = g.Dev(a), g.Dev(b)
        dst = da if target == 0 else db
        g.capi.check(name, da, db, 5000, dst, None)
        g.sync()
        g.assert_bf16_within(dst.get(), ref(a, b), 0 if exact else 1, 0.99, name)
        assert dst.guards_intact()


def test_pointwise_every_gate_pattern(g):
    gate = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    for up_bits in (0x3F80, 0xBFC0, 0x4049):
        up = np.full(65536, up_bits, dtype=np.uint16)
        dg, du = g.Dev(gate), g.Dev(up)
        out = g.empty_like_dev((65536,))
        g.capi.check("q3x_b200_silu_mul", dg, du, 65536, out, None)
        g.sync()
        g.assert_bf16_within(out.get(), orc.silu_mul(gate, up), 1, 0.995, "silu_mul sweep")
        g.capi.check("q3x_b200_sigmoid_gate", du, dg, 65536, out, None)
        g.sync()
        g.assert_bf16_within(out.get(), orc.sigmoid_gate(up, gate), 1, 0.995, "sigmoid_gate sweep")


@pytest.mark.parametrize("tokens,inter", [(1, 17408), (7, 17408), (33, 384), (5, 100)])
def test_silu_mul_merged(g, tokens, inter):
    rng = rng_for(tokens, inter, 3)
    merged = fx.normal_bf16(rng, (tokens, 2 * inter), 1.5)
    dm = g.Dev(merged)
    out = g.empty_like_dev((tokens, inter))
    g.capi.check("q3x_b200_silu_mul_merged", dm, tokens, inter, out, None)
    g.sync()
    g.assert_bf16_within(out.get(), orc.silu_mul_merged(merged), 1, 0.99, "merged SwiGLU")
    # and equal to the split-layout op on the same values
    dg = g.Dev(np.ascontiguousarray(merged[:, :inter]))
    du = g.Dev(np.ascontiguousarray(merged[:, inter:]))
    out2 = g.empty_like_dev((tokens, inter))
    g.capi.check("q3x_b200_silu_mul", dg, du, tokens * inter, out2, None)
    g.sync()
    g.assert_bits_equal(out.get(), out2.get(), "merged vs split SwiGLU")
    assert out.guards_intact()


def test_fp32_to_bf16(g):
    rng = rng_for(4)
    bits = np.concatenate([
        rng.integers(0, 2**32, size=100_000, dtype=np.uint64).astype(np.uint32),
        np.array([0x3F808000, 0x3F818000, 0, 0x80000000, 0x7F800000, 0xFF800000, 0x7F800001, 0xFFC00001,
                  0x7F7FFFFF, 1, 0x00008000], dtype=np.uint32)])
    vals = bits.view(np.float32)
    d = g.Dev(vals)
    out = g.empty_like_dev((vals.size,))
    g.capi.check("q3x_b200_fp32_to_bf16", d, vals.size, out, None)
    g.sync()
    g.assert_bits_equal(out.get(), orc.bf16_encode(vals), "fp32->bf16")  # NaN payload rule included


@pytest.mark.parametrize("heads,dim,misalign", [(24, 256, 0), (4, 8, 0), (3, 7, 0), (24, 256, 1), (512 * 24, 256, 0)])
def test_split_q_gate(g, heads, dim, misalign):
    rng = rng_for(heads, dim, 5)
    x = rng.integers(0, 65536, size=(heads, 2, dim), dtype=np.uint32).astype(np.uint16)
    dx = g.Dev(x, misalign)
    q, gate = g.empty_like_dev((heads, dim), misalign=misalign), g.empty_like_dev((heads, dim))
    g.capi.check("q3x_b200_split_interleaved_q_gate", dx, heads, dim, q, gate, None)
    g.sync()
    g.assert_bits_equal(q.get(), x[:, 0, :], "split q")
    g.assert_bits_equal(gate.get(), x[:, 1, :], "split gate")
    assert q.guards_intact() and gate.guards_intact()


# ----------------------------------------------------------------------------- norms

@pytest.mark.parametrize("rows,width,misalign", [
    (1, 5120, 0), (1, 777, 0), (1, 13, 0), (3, 256, 0), (24, 256, 0), (4, 256, 0), (48, 128, 0), (5, 127, 0),
    (33, 5120, 0), (512, 5120, 0), (7, 64, 0), (9, 384, 0), (2, 8192, 0), (2, 10000, 0), (5, 5120, 1), (6, 128, 2),
    (100_001, 128, 0)])
@pytest.mark.parametrize("centered", [True, False])
def test_rms_norm(g, rows, width, misalign, centered):
    rng = rng_for(rows, width, misalign, 6)
    x = fx.normal_bf16(rng, (rows, width))
    if rows * width > 5000:
        fx.sprinkle_specials(rng, x[-1:], 0.002)
    w = fx.normal_bf16(rng, (width,), 0.02 if centered else 1.0)
    dx, dw = g.Dev(x, misalign), g.Dev(w)
    out = g.empty_like_dev((rows, width), misalign=misalign)
    g.capi.check("q3x_b200_rms_norm", dx, dw, rows, width, EPS, int(centered), out, None)
    g.sync()
    g.assert_bf16_within(out.get(), orc.rms_norm_rows(x, w, EPS, centered), 1, 0.98, f"rms_norm {rows}x{width}")
    assert out.guards_intact()
    # in place
    g.capi.check("q3x_b200_rms_norm", dx, dw, rows, width, EPS, int(centered), dx, None)
    g.sync()
    g.assert_bits_equal(dx.get(), out.get(), "in-place rms_norm equals out-of-place")


@pytest.mark.parametrize("rows,width", [(48, 128), (5, 128), (8192 * 48 // 64, 128), (7, 256), (3, 100)])
def test_rms_norm_silu_gate(g, rows, width):
    rng = rng_for(rows, width, 7)
    x = fx.normal_bf16(rng, (rows, width))
    z = fx.normal_bf16(rng, (rows, width))
    w = orc.bf16_encode((0.75 + rng.random(width) * 0.5).astype(np.float32))
    dx, dz, dw = g.Dev(x), g.Dev(z), g.Dev(w)
    out = g.empty_like_dev((rows, width))
    g.capi.check("q3x_b200_rms_norm_silu_gate", dx, dw, dz, rows, width, EPS, out, None)
    g.sync()
    g.assert_bf16_within(out.get(), orc.rms_norm_rows(x, w, EPS, centered=False, gate=z), 1, 0.98, "gated norm")
    g.capi.check("q3x_b200_rms_norm_silu_gate", dx, dw, dz, rows, width, EPS, dx, None)  # in place on x
    g.sync()
    g.assert_bits_equal(dx.get(), out.get(), "in-place gated norm")
    assert out.guards_intact()


@pytest.mark.parametrize("heads,dim", [(5, 127), (16, 128), (5, 11), (8192 * 16, 128), (3, 256)])
@pytest.mark.parametrize("scale", [1.0, 0.08838834764831845])
def test_l2_normalize(g, heads, dim, scale):
    rng = rng_for(heads, dim, 8)
    x = fx.normal_bf16(rng, (heads, dim))
    x[0] = 0
    scale = float(np.float32(scale))
    dx = g.Dev(x)
    out = g.empty_like_dev((heads, dim))
    g.capi.check("q3x_b200_l2_normalize_heads", dx, heads, dim, EPS, scale, out, None)
    g.sync()
    g.assert_bf16_within(out.get(), orc.l2_normalize_heads(x, EPS, scale), 1, 0.98, "l2 norm")
    assert out.guards_intact()


def residual_fixture(kind, tokens, hidden, rng):
    """The three fixture families of the reference's fused residual/norm tests
    (tests/decode_ops_cuda_test.cu:1771-1826): structured, xorshift "random-like", non-finite."""
    n = tokens * hidden
    if kind == "structured":
        left = fx.structured_bf16(n, 41, 20, 8).reshape(tokens, hidden)
        right = fx.structured_bf16(n, 23, 11, 16).reshape(tokens, hidden)
    elif kind == "xorshift":
        m = min(n, 20480)
        left = np.resize(fx.xorshift_bf16(m, 0x9E3779B9), n).reshape(tokens, hidden)
        right = np.resize(fx.xorshift_bf16(m, 0x85EBCA6B), n).reshape(tokens, hidden)
    else:
        left = fx.normal_bf16(rng, (tokens, hidden))
        right = fx.normal_bf16(rng, (tokens, hidden))
        if kind == "nonfinite":
            fx.sprinkle_specials(rng, left, 0.0005)
            fx.sprinkle_specials(rng, right, 0.0005)
    return left, right


@pytest.mark.parametrize("tokens", [1, 2, 7, 31, 32, 33, 407, 511, 512, 513])
@pytest.mark.parametrize("kind", ["normal", "structured", "xorshift", "nonfinite"])
def test_residual_add_rms_norm(g, tokens, kind):
    if kind != "normal" and tokens not in (1, 32, 33, 512):
        pytest.skip("fixture families run on a subset of tile sizes")
    hidden = 5120
    rng = rng_for(tokens, kind, 9)
    left, right = residual_fixture(kind, tokens, hidden, rng)
    w = fx.normal_bf16(rng, (hidden,), 0.02)
    dl, dr, dw = g.Dev(left), g.Dev(right), g.Dev(w)
    res, nrm = g.empty_like_dev((tokens, hidden)), g.empty_like_dev((tokens, hidden))
    g.capi.check("q3x_b200_residual_add_rms_norm", dl, dr, dw, tokens, hidden, EPS, res, nrm, None)
    g.sync()
    want_r, want_n = orc.residual_add_rms_norm(left, right, w, EPS)
    nan = orc.bf16_is_nan(want_r)
    g.assert_bits_equal(res.get()[~nan], want_r[~nan], "residual (bit-exact)")
    g.assert_bf16_within(nrm.get(), want_n, 1, 0.98, "normalized")
    assert res.guards_intact() and nrm.guards_intact()
    # fused == the two-op chain on the GPU, bit for bit (include/q3x/runtime/decode_ops.h:230-234)
    r2, n2 = g.empty_like_dev((tokens, hidden)), g.empty_like_dev((tokens, hidden))
    g.capi.check("q3x_b200_residual_add", dl, dr, tokens * hidden, r2, None)
    g.capi.check("q3x_b200_rms_norm", r2, dw, tokens, hidden, EPS, 1, n2, None)
    g.sync()
    g.assert_bits_equal(r2.get(), res.get(), "fused residual == unfused")
    g.assert_bits_equal(n2.get(), nrm.get(), "fused normalized == unfused")
    # normalized may alias right exactly; NULL normalized is allowed
    g.capi.check("q3x_b200_residual_add_rms_norm", dl, dr, dw, tokens, hidden, EPS, r2, dr, None)
    g.sync()
    g.assert_bits_equal(dr.get(), nrm.get(), "normalized aliasing right")
    r3 = g.empty_like_dev((tokens, hidden))
    dr2 = g.Dev(right)
    g.capi.check("q3x_b200_residual_add_rms_norm", dl, dr2, dw, tokens, hidden, EPS, r3, None, None)
    g.sync()
    g.assert_bits_equal(r3.get(), res.get(), "residual only")


@pytest.mark.parametrize("tokens,hidden,misalign", [(3, 777, 0), (5, 5120, 1), (4, 64, 0), (2, 9000, 0)])
def test_residual_add_rms_norm_other_shapes(g, tokens, hidden, misalign):
    rng = rng_for(tokens, hidden, 10)
    left, right = fx.normal_bf16(rng, (tokens, hidden)), fx.normal_bf16(rng, (tokens, hidden))
    w = fx.normal_bf16(rng, (hidden,), 0.02)
    dl, dr, dw = g.Dev(left, misalign), g.Dev(right, misalign), g.Dev(w)
    res, nrm = g.empty_like_dev((tokens, hidden), misalign=misalign), g.empty_like_dev((tokens, hidden))
    g.capi.check("q3x_b200_residual_add_rms_norm", dl, dr, dw, tokens, hidden, EPS, res, nrm, None)
    g.sync()
    want_r, want_n = orc.residual_add_rms_norm(left, right, w, EPS)
    g.assert_bits_equal(res.get(), want_r, "residual")
    g.assert_bf16_within(nrm.get(), want_n, 1, 0.98, "normalized")
    assert res.guards_intact() and nrm.guards_intact()


# ----------------------------------------------------------------------------- full attention

@pytest.mark.parametrize("tokens,first", [(1, 4096), (2, 0), (8, 17), (16, 33), (32, 0), (407, 5), (512, 0), (513, 100)])
def test_full_attention_preprocess(g, tokens, first):
    rng = rng_for(tokens, first, 11)
    qg = fx.normal_bf16(rng, (tokens, 24, 2, 256))
    key = fx.normal_bf16(rng, (tokens, 4, 256))
    if tokens >= 8:
        fx.sprinkle_specials(rng, qg[-1:], 0.001)
    qw, kw = fx.normal_bf16(rng, (256,), 0.02), fx.normal_bf16(rng, (256,), 0.02)
    cos, sin = orc.rope_tables(0, first + tokens)
    d_qg, d_key, d_qw, d_kw = g.Dev(qg), g.Dev(key), g.Dev(qw), g.Dev(kw)
    d_cos, d_sin = g.Dev(cos), g.Dev(sin)
    q, gate = g.empty_like_dev((tokens, 24, 256)), g.empty_like_dev((tokens, 24, 256))
    g.capi.check("q3x_b200_full_attention_preprocess", d_qg, d_key, d_qw, d_kw, EPS, q, gate, d_cos, d_sin, first,
                 tokens, None)
    g.sync()
    want_q, want_g, want_k = orc.full_attention_preprocess(qg, key, qw, kw, EPS, cos, sin, first)
    g.assert_bits_equal(gate.get(), want_g, "gate is a raw copy")
    assert q.guards_intact() and gate.guards_intact() and d_key.guards_intact()
    assert np.array_equal(d_qg.get(), qg)
    # The op is two roundings in a row (head norm -> bf16 -> rotation -> bf16).  Where the first
    # rounding lands one ulp away from the host's, the rotation's subtraction can amplify it, so
    # the 1-ulp bound is checked per stage on identical operands, and the whole chain end to end on
    # the pass-through dims (one rounding) plus an exact-match quota on the rotated ones.
    q2, g2 = g.empty_like_dev((tokens, 24, 256)), g.empty_like_dev((tokens, 24, 256))
    k2 = g.Dev(key)
    g.capi.check("q3x_b200_split_interleaved_q_gate", d_qg, tokens * 24, 256, q2, g2, None)
    g.capi.check("q3x_b200_rms_norm", q2, d_qw, tokens * 24, 256, EPS, 1, q2, None)
    g.capi.check("q3x_b200_rms_norm", k2, d_kw, tokens * 4, 256, EPS, 1, k2, None)
    g.sync()
    q_normed, k_normed = q2.get(), k2.get()
    g.assert_bf16_within(q_normed, orc.rms_norm_rows(qg[:, :, 0, :], qw, EPS), 1, 0.98, "q head norm")
    g.assert_bf16_within(k_normed, orc.rms_norm_rows(key, kw, EPS), 1, 0.98, "k head norm")
    g.capi.check("q3x_b200_qk_partial_neox_rope", q2, k2, d_cos, d_sin, first, tokens, None)
    g.sync()
    # stage 2 on the GPU's own rounded operand: bit-exact against the host rotation
    for t in (0, tokens // 2, tokens - 1):
        g.assert_bf16_within(q2.get()[t], orc.partial_rope(q_normed[t], cos[first + t], sin[first + t]), 0, 1.0,
                             "rotation of q")
        g.assert_bf16_within(k2.get()[t], orc.partial_rope(k_normed[t], cos[first + t], sin[first + t]), 0, 1.0,
                             "rotation of k")
    # the fused pass equals split -> head norm -> RoPE run as separate launches, bit for bit
    g.assert_bits_equal(q2.get(), q.get(), "fused q == unfused chain")
    g.assert_bits_equal(k2.get(), d_key.get(), "fused k == unfused chain")
    # end to end against the host chain
    g.assert_bf16_within(q.get()[:, :, 64:], want_q[:, :, 64:], 1, 0.98, "q pass-through dims")
    g.assert_bf16_within(d_key.get()[:, :, 64:], want_k[:, :, 64:], 1, 0.98, "k pass-through dims")
    _, exact_q = g.ulp_report(q.get()[:, :, :64], want_q[:, :, :64])
    _, exact_k = g.ulp_report(d_key.get()[:, :, :64], want_k[:, :, :64])
    assert exact_q > 0.97 and exact_k > 0.97
    # hard bound on the rotated dims end to end: the reference's own tolerance for this operator
    g.assert_reference_tolerance(q.get(), want_q, "q end to end", amplified=True)
    g.assert_reference_tolerance(d_key.get(), want_k, "k end to end", amplified=True)


@pytest.mark.parametrize("heads,misalign", [(3, 0), (28, 0), (24, 1)])
def test_partial_rope_single_position(g, heads, misalign):
    rng = rng_for(heads, 12)
    x = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (heads, 256)), 0.005)
    cos, sin = orc.rope_tables(4096, 1)
    dx, dc, ds = g.Dev(x, misalign), g.Dev(cos), g.Dev(sin)
    out = g.empty_like_dev((heads, 256), misalign=misalign)
    g.capi.check("q3x_b200_partial_neox_rope_256_64", dx, dc, ds, heads, out, None)
    g.sync()
    want = orc.partial_rope(x, cos[0], sin[0])
    # same un-fused multiply / add as the host op: expected bit-exact
    g.assert_bf16_within(out.get(), want, 0, 1.0, "partial rope")
    g.capi.check("q3x_b200_partial_neox_rope_256_64", dx, dc, ds, heads, dx, None)
    g.sync()
    g.assert_bits_equal(dx.get(), out.get(), "in-place rope")
    assert out.guards_intact()


# ----------------------------------------------------------------------------- GDN conv

CONV_TOKENS = [1, 2, 3, 7, 8, 9, 31, 32, 33, 64, 407, 513]


@pytest.mark.parametrize("tokens", CONV_TOKENS)
def test_causal_conv(g, tokens):
    rng = rng_for(tokens, 13)
    C_ = 10240
    raw = fx.normal_bf16(rng, (tokens, C_))
    if tokens > 8:
        fx.sprinkle_specials(rng, raw[3:4], 0.001)
    w = fx.normal_bf16(rng, (C_, 4), 0.5)
    hist = fx.normal_bf16(rng, (C_, 3))
    d_raw, d_w, d_h = g.Dev(raw), g.Dev(w), g.Dev(hist)
    out = g.empty_like_dev((tokens, C_))
    g.capi.check("q3x_b200_causal_conv1d_silu", d_raw, tokens, C_, d_w, d_h, out, None)
    g.sync()
    want, want_h = orc.causal_conv1d_silu(raw, w, hist)
    g.assert_bf16_within(out.get(), want, 1, 0.985, "conv")
    g.assert_bits_equal(d_h.get(), want_h, "history holds the last raw rows")
    assert out.guards_intact() and d_h.guards_intact() and np.array_equal(d_raw.get(), raw)
    # in place (serial path) gives the same bits as the token-parallel path
    d_h2 = g.Dev(hist)
    g.capi.check("q3x_b200_causal_conv1d_silu", d_raw, tokens, C_, d_w, d_h2, d_raw, None)
    g.sync()
    g.assert_bits_equal(d_raw.get(), out.get(), "in-place conv == out-of-place")
    g.assert_bits_equal(d_h2.get(), want_h, "history (in place)")


def test_causal_conv_chunks_chain_through_history(g):
    rng = rng_for(14)
    C_, T = 10240, 100
    raw = fx.normal_bf16(rng, (T, C_))
    w = fx.normal_bf16(rng, (C_, 4), 0.5)
    zero = np.zeros((C_, 3), dtype=np.uint16)
    d_w = g.Dev(w)
    whole = g.empty_like_dev((T, C_))
    h1 = g.Dev(zero)
    g.capi.check("q3x_b200_causal_conv1d_silu", g.Dev(raw), T, C_, d_w, h1, whole, None)
    pieces = g.empty_like_dev((T, C_))
    h2 = g.Dev(zero)
    d_raw = g.Dev(raw)
    start = 0
    for n in (1, 2, 37, 60):
        g.capi.check("q3x_b200_causal_conv1d_silu", d_raw.ptr_at(start * C_), n, C_, d_w, h2,
                     pieces.ptr_at(start * C_), None)
        start += n
    g.sync()
    g.assert_bits_equal(pieces.get(), whole.get(), "chunked conv == whole-span conv")
    g.assert_bits_equal(h2.get(), h1.get(), "history after chunks")


@pytest.mark.parametrize("tokens", [1, 5, 33, 130])
def test_causal_conv_l2norm(g, tokens):
    rng = rng_for(tokens, 15)
    C_ = 10240
    raw = fx.normal_bf16(rng, (tokens, C_))
    w = fx.normal_bf16(rng, (C_, 4), 0.5)
    hist = fx.normal_bf16(rng, (C_, 3))
    qs = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    d_raw, d_w, d_h = g.Dev(raw), g.Dev(w), g.Dev(hist)
    out = g.empty_like_dev((tokens, C_))
    g.capi.check("q3x_b200_causal_conv1d_silu_l2norm", d_raw, tokens, d_w, d_h, EPS, qs, out, None)
    # the same thing as two launches on the GPU must agree bit for bit
    plain = g.empty_like_dev((tokens, C_))
    d_h2 = g.Dev(hist)
    g.capi.check("q3x_b200_causal_conv1d_silu", d_raw, tokens, C_, d_w, d_h2, plain, None)
    g.sync()
    conv = plain.get()
    got = out.get()
    g.assert_bits_equal(got[:, 4096:], conv[:, 4096:], "v channels are the plain conv")
    # oracle chain on the GPU's own rounded conv output
    want_q = orc.l2_normalize_heads(conv[:, :2048].reshape(tokens * 16, 128), EPS, qs).reshape(tokens, 2048)
    want_k = orc.l2_normalize_heads(conv[:, 2048:4096].reshape(tokens * 16, 128), EPS, 1.0).reshape(tokens, 2048)
    g.assert_bf16_within(got[:, :2048], want_q, 1, 0.98, "q heads")
    g.assert_bf16_within(got[:, 2048:4096], want_k, 1, 0.98, "k heads")
    # and end to end against the CPU chain
    cpu_conv, want_h = orc.causal_conv1d_silu(raw, w, hist)
    cq = orc.l2_normalize_heads(cpu_conv[:, :2048].reshape(-1, 128), EPS, qs).reshape(tokens, 2048)
    worst, exact = g.ulp_report(got[:, :2048], cq)
    assert worst <= 2 and exact > 0.97  # two roundings in a row: each within 1 ulp
    ck = orc.l2_normalize_heads(cpu_conv[:, 2048:4096].reshape(-1, 128), EPS, 1.0).reshape(tokens, 2048)
    g.assert_reference_tolerance(got[:, :2048], cq, "conv -> L2 (q) end to end")
    g.assert_reference_tolerance(got[:, 2048:4096], ck, "conv -> L2 (k) end to end")
    g.assert_bits_equal(d_h.get(), want_h, "history")
    assert out.guards_intact()


# ----------------------------------------------------------------------------- embedding

@pytest.mark.parametrize("tokens", [1, 2, 7, 8, 31, 32, 64, 407, 481, 511, 512, 4099])
def test_embedding(g, tokens):
    rng = rng_for(tokens, 16)
    vocab, hidden = 1000, 5120
    table = rng.integers(0, 65536, size=(vocab, hidden), dtype=np.uint32).astype(np.uint16)
    ids = rng.integers(0, vocab, size=tokens, dtype=np.uint32)
    ids[0] = vocab - 1
    if tokens > 2:
        ids[1] = 0
        ids[2] = ids[0]  # repeated id
    bad = tokens > 7
    if bad:
        ids[5] = vocab + 3  # outside the vocabulary: row stays untouched
    d_t, d_i = g.Dev(table), g.Dev(ids)
    out = g.empty_like_dev((tokens, hidden), fill=0xABCD)
    g.capi.check("q3x_b200_embedding_gather", d_t, vocab, hidden, d_i, tokens, out, None)
    g.sync()
    want = orc.embedding_gather(table, ids, out=np.full((tokens, hidden), 0xABCD, dtype=np.uint16))
    g.assert_bits_equal(out.get(), want, "embedding rows")
    if bad:
        assert np.all(out.get()[5] == 0xABCD)
    assert out.guards_intact()


def test_embedding_odd_width_and_alignment(g):
    rng = rng_for(17)
    table = rng.integers(0, 65536, size=(5, 7), dtype=np.uint32).astype(np.uint16)
    ids = np.array([3, 0, 4, 4, 1], dtype=np.uint32)
    out = g.empty_like_dev((5, 7))
    g.capi.check("q3x_b200_embedding_gather", g.Dev(table), 5, 7, g.Dev(ids), 5, out, None)
    g.sync()
    g.assert_bits_equal(out.get(), table[ids], "7-wide rows")
    table = rng.integers(0, 65536, size=(9, 64), dtype=np.uint32).astype(np.uint16)
    out = g.empty_like_dev((5, 64), misalign=1)
    g.capi.check("q3x_b200_embedding_gather", g.Dev(table, 1), 9, 64, g.Dev(ids), 5, out, None)
    g.sync()
    g.assert_bits_equal(out.get(), table[ids], "misaligned rows")


# ----------------------------------------------------------------------------- golden fixtures

def test_against_golden_fixtures(g):
    """Outputs of the reference project's own host ops (tests/golden/make_golden.py)."""
    import os

    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_ops.npz"))
    res, nrm = g.empty_like_dev((6, 5120)), g.empty_like_dev((6, 5120))
    g.capi.check("q3x_b200_residual_add_rms_norm", g.Dev(gold["rn_left"]), g.Dev(gold["rn_right"]),
                 g.Dev(gold["rn_weight"]), 6, 5120, EPS, res, nrm, None)
    out = g.empty_like_dev((777,))
    results = {}
    for name, key in (("q3x_b200_residual_add", "pw_residual_want"), ("q3x_b200_silu_mul", "pw_silu_mul_want"),
                      ("q3x_b200_sigmoid_gate", "pw_sigmoid_gate_want")):
        g.capi.check(name, g.Dev(gold["pw_a"]), g.Dev(gold["pw_b"]), 777, out, None)
        g.sync()
        results[key] = out.get()
    hn = g.empty_like_dev((28, 256))
    g.capi.check("q3x_b200_rms_norm", g.Dev(gold["hn_x"]), g.Dev(gold["hn_w"]), 28, 256, EPS, 1, hn, None)
    gn = g.empty_like_dev((48, 128))
    g.capi.check("q3x_b200_rms_norm_silu_gate", g.Dev(gold["gn_x"]), g.Dev(gold["gn_w"]), g.Dev(gold["gn_z"]), 48, 128,
                 EPS, gn, None)
    l2a, l2b = g.empty_like_dev((16, 128)), g.empty_like_dev((5, 127))
    g.capi.check("q3x_b200_l2_normalize_heads", g.Dev(gold["l2a_x"]), 16, 128, EPS, 1.0, l2a, None)
    g.capi.check("q3x_b200_l2_normalize_heads", g.Dev(gold["l2b_x"]), 5, 127, EPS, 1.0, l2b, None)
    rope = g.empty_like_dev((28, 256))
    g.capi.check("q3x_b200_partial_neox_rope_256_64", g.Dev(gold["rope_x"]), g.Dev(gold["rope_cos"]),
                 g.Dev(gold["rope_sin"]), 28, rope, None)
    conv = g.empty_like_dev((4, 10240))
    hist = g.Dev(gold["conv_hist"])
    g.capi.check("q3x_b200_causal_conv1d_silu", g.Dev(gold["conv_raw"]), 4, 10240, g.Dev(gold["conv_w"]), hist, conv,
                 None)
    g.sync()
    nan = orc.bf16_is_nan(gold["rn_residual_want"])
    g.assert_bits_equal(res.get()[~nan], gold["rn_residual_want"][~nan], "golden residual")
    g.assert_bf16_within(nrm.get(), gold["rn_normalized_want"], 1, 0.98, "golden normalized")
    nan = orc.bf16_is_nan(gold["pw_residual_want"])
    g.assert_bits_equal(results["pw_residual_want"][~nan], gold["pw_residual_want"][~nan], "golden residual add")
    g.assert_bf16_within(results["pw_silu_mul_want"], gold["pw_silu_mul_want"], 1, 0.98, "golden silu_mul")
    g.assert_bf16_within(results["pw_sigmoid_gate_want"], gold["pw_sigmoid_gate_want"], 1, 0.98, "golden sigmoid")
    g.assert_bf16_within(hn.get(), gold["hn_centered_want"], 1, 0.98, "golden head norm")
    g.assert_bf16_within(gn.get(), gold["gn_want"], 1, 0.98, "golden gated norm")
    g.assert_bf16_within(l2a.get(), gold["l2a_want"], 1, 0.98, "golden l2 16x128")
    g.assert_bf16_within(l2b.get(), gold["l2b_want"], 1, 0.98, "golden l2 5x127")
    g.assert_bf16_within(rope.get(), gold["rope_want"], 0, 1.0, "golden rope")
    g.assert_bf16_within(conv.get(), gold["conv_want"], 1, 0.98, "golden conv")
    g.assert_bits_equal(hist.get(), gold["conv_hist_want"], "golden conv history")
