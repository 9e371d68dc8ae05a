"""Pins the C restatement (oracle/q3x_oracle.c) against the reference project's own host
reference ops compiled from its sources (oracle/_ref/libq3x_ref.so): bit-for-bit, on seeded
random inputs, on special values and on the deterministic fixtures of the reference's own tests.

Skipped where ``oracle/_ref`` was never built (no reference checkout at build time); the
committed fixtures under tests/golden/ cover that case (test_oracle_golden.py).
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tests import fixtures as fx

pytestmark = pytest.mark.skipif(not orc.have_ref(), reason="oracle/_ref not built")

EPS = 1e-6
u16p = C.POINTER(C.c_uint16)
f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)


def p(a, ty=u16p):
    return a.ctypes.data_as(ty)


def same(a, b):
    """Bit equality, except that any NaN equals any NaN: which operand's payload and sign a
    NaN result inherits depends on the compiler's operand order, not on the algorithm."""
    return bool(np.all(orc.bf16_ulp_distance(a, b) == 0) and
                np.array_equal(orc.bf16_is_nan(a), orc.bf16_is_nan(b)) and
                np.array_equal(np.asarray(a)[~orc.bf16_is_nan(a)], np.asarray(b)[~orc.bf16_is_nan(b)]))


@pytest.fixture(scope="module")
def ref():
    orc.build()
    return orc.ref_lib()


def rows_with_specials(seed, shape):
    rng = np.random.default_rng(seed)
    return fx.sprinkle_specials(rng, fx.normal_bf16(rng, shape))


def test_bf16_encode_matches_reference_on_every_interesting_float(ref):
    rng = np.random.default_rng(1)
    bits = np.concatenate([
        rng.integers(0, 2**32, size=200_000, dtype=np.uint64).astype(np.uint32),
        np.array([0x3F808000, 0x3F818000, 0, 0x80000000, 0x7F800000, 0xFF800000, 0x7F800001, 0x7FFFFFFF,
                  0xFF800001, 0x7F7FFFFF, 0x00000001, 0x00008000, 0x00018000], dtype=np.uint32),
    ])
    vals = bits.view(np.float32)
    want = np.empty(vals.size, dtype=np.uint16)
    assert ref.fp32_to_bf16(p(vals, f32p), vals.size, p(want)) == 0
    assert np.array_equal(orc.bf16_encode(vals), want)
    got = np.empty(vals.size, dtype=np.uint16)
    assert orc.oracle_lib().fp32_to_bf16(p(vals, f32p), vals.size, p(got)) == 0
    assert np.array_equal(got, want)
    # the reference's own known answers (tests/decode_ops_host_test.cpp:456-478)
    known = dict(zip(bits[-13:-6].tolist(), want[-13:-6].tolist()))
    assert known[0x3F808000] == 0x3F80 and known[0x3F818000] == 0x3F82
    assert known[0] == 0x0000 and known[0x80000000] == 0x8000
    assert known[0x7F800000] == 0x7F80 and known[0xFF800000] == 0xFF80
    assert known[0x7F800001] & 0x7FC0 == 0x7FC0


@pytest.mark.parametrize("width", [1, 7, 13, 128, 256, 777, 5120])
@pytest.mark.parametrize("centered", [True, False])
def test_rms_norm(ref, width, centered):
    x = rows_with_specials(width, (width,)) if width > 100 else fx.normal_bf16(np.random.default_rng(width), (width,))
    w = fx.normal_bf16(np.random.default_rng(2), (width,), 0.02)
    want = np.empty_like(x)
    fn = ref.centered if centered else ref.plain
    assert fn(p(x), p(w), width, EPS, p(want)) == 0
    got = np.empty_like(x)
    assert orc.oracle_lib().rms_norm(p(x), p(w), width, EPS, int(centered), p(got)) == 0
    assert same(got, want)


@pytest.mark.parametrize("heads,dim", [(3, 256), (24, 256), (4, 256), (48, 128), (5, 127), (33, 5120)])
def test_headwise_norms(ref, heads, dim):
    rng = np.random.default_rng(heads * 1000 + dim)
    x = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (heads, dim)), 0.002)
    g = fx.normal_bf16(rng, (heads, dim))
    w = fx.normal_bf16(rng, (dim,), 0.02)
    want = np.empty_like(x)
    assert ref.head_centered(p(x), p(w), heads, dim, EPS, p(want)) == 0
    assert same(orc.rms_norm_rows(x, w, EPS, centered=True), want)
    assert ref.head_plain(p(x), p(w), heads, dim, EPS, p(want)) == 0
    assert same(orc.rms_norm_rows(x, w, EPS, centered=False), want)
    assert ref.head_plain_gate(p(x), p(w), p(g), heads, dim, EPS, p(want)) == 0
    assert same(orc.rms_norm_rows(x, w, EPS, centered=False, gate=g), want)


def test_reference_headwise_fixture(ref):
    """The structured fixture of tests/decode_ops_host_test.cpp:323-414, regenerated."""
    i = np.arange(3 * 256)
    x = orc.bf16_encode((((i * 7) % 41) - 20).astype(np.float32) / (8 + i // 256).astype(np.float32))
    w = orc.bf16_encode(((np.arange(256) % 9) - 4).astype(np.float32) / np.float32(32))
    want = np.empty_like(x)
    assert ref.head_centered(p(x), p(w), 3, 256, EPS, p(want)) == 0
    got = orc.rms_norm_rows(x.reshape(3, 256), w, EPS).reshape(-1)
    assert np.array_equal(got, want)
    xd = orc.bf16_decode(x).astype(np.float64).reshape(3, 256)
    exp = xd / np.sqrt((xd**2).mean(-1, keepdims=True) + EPS) * (1 + orc.bf16_decode(w).astype(np.float64))
    err = np.abs(orc.bf16_decode(got).reshape(3, 256) - exp)
    assert np.all(err <= np.maximum(2e-3, 8e-3 * np.abs(exp)))  # the reference's own tolerance


@pytest.mark.parametrize("count", [17, 777, 100_003])
def test_pointwise(ref, count):
    a = rows_with_specials(count, (count,))
    b = rows_with_specials(count + 1, (count,))
    want = np.empty_like(a)
    assert ref.residual_add(p(a), p(b), count, p(want)) == 0
    assert same(orc.residual_add(a, b), want)
    assert ref.silu_mul(p(a), p(b), count, p(want)) == 0
    assert same(orc.silu_mul(a, b), want)
    assert ref.sigmoid_gate(p(a), p(b), count, p(want)) == 0
    assert same(orc.sigmoid_gate(a, b), want)


def test_pointwise_every_gate_bit_pattern(ref):
    """All 65536 bf16 gate values against a handful of multiplicands."""
    gate = np.arange(65536, dtype=np.uint16)
    for up_bits in (0x3F80, 0xBFC0, 0x0000, 0x7F80, 0x4049):
        up = np.full(65536, up_bits, dtype=np.uint16)
        want = np.empty_like(gate)
        assert ref.silu_mul(p(gate), p(up), 65536, p(want)) == 0
        assert same(orc.silu_mul(gate, up), want)
        assert ref.sigmoid_gate(p(up), p(gate), 65536, p(want)) == 0
        assert same(orc.sigmoid_gate(up, gate), want)


def test_residual_add_rms_norm_chain(ref):
    rng = np.random.default_rng(5)
    left = fx.normal_bf16(rng, (9, 5120))
    right = fx.normal_bf16(rng, (9, 5120))
    w = fx.normal_bf16(rng, (5120,), 0.02)
    res, nrm = orc.residual_add_rms_norm(left, right, w, EPS)
    want_r = np.empty_like(left)
    want_n = np.empty_like(left)
    assert ref.residual_add(p(left), p(right), left.size, p(want_r)) == 0
    assert ref.head_centered(p(want_r), p(w), 9, 5120, EPS, p(want_n)) == 0
    assert np.array_equal(res, want_r) and np.array_equal(nrm, want_n)


@pytest.mark.parametrize("heads,dim", [(5, 11), (5, 127), (16, 128), (8192, 128)])
def test_l2_normalize(ref, heads, dim):
    rng = np.random.default_rng(heads + dim)
    x = fx.normal_bf16(rng, (heads, dim))
    x[0, :] = 0  # an all-zero head exercises the epsilon
    want = np.empty_like(x)
    assert ref.l2(p(x), heads, dim, EPS, p(want)) == 0
    assert np.array_equal(orc.l2_normalize_heads(x, EPS), want)


def test_rope_and_tables(ref):
    rng = np.random.default_rng(11)
    x = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (28, 256)), 0.003)
    cos, sin = orc.rope_tables(4096, 3)
    # the table recipe, restated with numpy float32 (src/runtime/request_state.cpp:2092-2108)
    pair = np.arange(32, dtype=np.float32)
    inv = np.float32(1.0) / np.power(np.float32(1e7), np.float32(2.0) * pair / np.float32(64.0)).astype(np.float32)
    for r, pos in enumerate((4096, 4097, 4098)):
        ang = (np.float32(pos) * inv).astype(np.float32)
        # libm float cos/sin vs numpy's may differ in the last bit; after the bf16 round trip
        # they must agree except on rare boundary cases
        assert np.mean(orc.bf16_encode(np.cos(ang)) == orc.bf16_encode(cos[r])) > 0.9
        assert np.array_equal(orc.bf16_decode(orc.bf16_encode(cos[r])), cos[r])
        assert np.array_equal(orc.bf16_decode(orc.bf16_encode(sin[r])), sin[r])
    want = np.empty_like(x)
    assert ref.rope(p(x), p(cos[1], f32p), p(sin[1], f32p), 28, p(want)) == 0
    assert same(orc.partial_rope(x, cos[1], sin[1]), want)
    assert np.array_equal(want[:, 64:], x[:, 64:])


def test_split_and_preprocess_chain(ref):
    rng = np.random.default_rng(12)
    tokens, first = 5, 37
    qg = fx.normal_bf16(rng, (tokens, 24, 2, 256))
    key = fx.normal_bf16(rng, (tokens, 4, 256))
    qw = fx.normal_bf16(rng, (256,), 0.02)
    kw = fx.normal_bf16(rng, (256,), 0.02)
    cos, sin = orc.rope_tables(0, first + tokens)
    q, g, k = orc.full_attention_preprocess(qg, key, qw, kw, EPS, cos, sin, first)
    for t in range(tokens):
        wq = np.empty(24 * 256, dtype=np.uint16)
        wg = np.empty(24 * 256, dtype=np.uint16)
        row = np.ascontiguousarray(qg[t]).reshape(-1)
        assert ref.split(p(row), 24, 256, p(wq), p(wg)) == 0
        assert np.array_equal(g[t].reshape(-1), wg)
        assert np.array_equal(wq.reshape(24, 256), qg[t, :, 0, :])
        assert ref.head_centered(p(wq), p(qw), 24, 256, EPS, p(wq)) == 0
        assert ref.rope(p(wq), p(cos[first + t], f32p), p(sin[first + t], f32p), 24, p(wq)) == 0
        assert np.array_equal(q[t].reshape(-1), wq)
        wk = np.ascontiguousarray(key[t]).reshape(-1).copy()
        assert ref.head_centered(p(wk), p(kw), 4, 256, EPS, p(wk)) == 0
        assert ref.rope(p(wk), p(cos[first + t], f32p), p(sin[first + t], f32p), 4, p(wk)) == 0
        assert np.array_equal(k[t].reshape(-1), wk)


def test_split_rejects_overlap(ref):
    buf = np.zeros(4 * 2 * 8 + 64, dtype=np.uint16)
    L = orc.oracle_lib()
    q = buf[8:8 + 32]
    assert L.split(p(buf), 4, 8, p(q), p(buf[64:])) == orc.STATUS_INVALID_ALIAS
    assert ref.split(p(buf), 4, 8, p(q), p(buf[64:])) != 0


@pytest.mark.parametrize("tokens", [1, 2, 3, 7, 33])
def test_causal_conv(ref, tokens):
    rng = np.random.default_rng(tokens)
    C_ = 10240
    raw = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (tokens, C_)), 0.001)
    w = fx.normal_bf16(rng, (C_, 4), 0.5)
    hist = fx.normal_bf16(rng, (C_, 3))
    out, new_hist = orc.causal_conv1d_silu(raw, w, hist)
    h = hist.copy()
    for t in range(tokens):
        want = np.empty(C_, dtype=np.uint16)
        row = np.ascontiguousarray(raw[t])
        assert ref.conv(p(row), p(w), p(h), p(want)) == 0
        assert same(out[t], want), t
    assert np.array_equal(new_hist, h)


def test_conv_orientation_fixture(ref):
    """tests/gdn_decode_host_test.cpp:174-217: weights 1,2,4,8 oldest->newest on one channel."""
    C_ = 10240
    w = np.zeros((C_, 4), dtype=np.uint16)
    w[173] = orc.bf16_encode(np.array([1, 2, 4, 8], dtype=np.float32))
    raw = np.zeros((5, C_), dtype=np.uint16)
    raw[:, 173] = orc.bf16_encode((np.arange(5) + 1).astype(np.float32) * np.float32(0.25))
    out, hist = orc.causal_conv1d_silu(raw, w, np.zeros((C_, 3), dtype=np.uint16))
    e = [0.0, 0.0, 0.0]
    for s in range(5):
        cur = (s + 1) * 0.25
        conv = np.float32(e[0] + 2 * e[1] + 4 * e[2] + 8 * cur)
        silu = np.float32(conv / (np.float32(1) + np.exp(-conv, dtype=np.float32)))
        assert abs(float(orc.bf16_decode(out[s, 173])) - float(silu)) <= 8e-3 * abs(float(silu)) + 1e-6
        e = [e[1], e[2], cur]
    assert np.array_equal(orc.bf16_decode(hist[173]), np.array(e, dtype=np.float32))


def test_nvfp4_primitives_every_code(ref):
    L = orc.oracle_lib()
    for n in range(16):
        a, b = L.decode_e2m1(n), ref.decode_e2m1(n)
        assert a == b and np.signbit(a) == np.signbit(b)
    for c in range(256):
        a, b = L.decode_e4m3(c), ref.decode_e4m3(c)
        assert (np.isnan(a) and np.isnan(b)) or (a == b and np.signbit(a) == np.signbit(b)), c
    for byte in (0x00, 0x1F, 0xA5, 0xF0):
        assert ref.unpack(byte, 0) == byte & 0xF and ref.unpack(byte, 1) == byte >> 4


def test_e4m3_encoder_equals_reference_quantiser_on_every_bf16(ref):
    """The reference's E4M3 activation quantiser (gemv_reference.cpp:35-62), observed through
    its static W8A8 GEMV with scale 1, against decode(encode(x)) for all 65536 bf16 inputs."""
    L = orc.oracle_lib()
    out = C.c_float()
    for bits in range(65536):
        x = float(orc.bf16_decode(np.uint16(bits)))
        if np.isnan(x):
            continue
        assert ref.e4m3_value(bits, 1.0, C.byref(out)) == 0
        got = L.decode_e4m3(L.encode_e4m3(x))
        assert got == out.value, (hex(bits), x, got, out.value)


def test_nvfp4_round_trip_through_reference_dequantiser(ref):
    rng = np.random.default_rng(21)
    x = fx.normal_bf16(rng, (40, 5120))
    codes, scales, gs = orc.nvfp4_quantize(x, rows_per_scale=16)
    for g in range(3):
        rows = slice(g * 16, min(40, g * 16 + 16))
        want = np.empty((codes[rows].shape[0], 5120), dtype=np.float32)
        c = np.ascontiguousarray(codes[rows])
        s = np.ascontiguousarray(scales[rows])
        assert ref.dequant(p(c, u8p), p(s, u8p), float(gs[g]), c.shape[0], 5120, p(want, f32p)) == 0
        assert np.array_equal(orc.nvfp4_dequantize(c, s, gs[g]), want)
        xf = orc.bf16_decode(x[rows])
        # every element is reproduced to within half an E2M1 step of its block scale
        block_d = np.repeat(np.array([orc.oracle_lib().decode_e4m3(int(v)) for v in s.reshape(-1)],
                                     dtype=np.float32).reshape(s.shape), 16, axis=1) * gs[g]
        assert np.all(np.abs(want - xf) <= block_d * 1.0 + 1e-12)
