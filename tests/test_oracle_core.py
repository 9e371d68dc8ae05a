"""The CPU restatement of the operators BETWEEN the fused layer ops (q3x_oracle_core.c: gated-delta-net
recurrence, softmax, GQA attention, greedy argmax, batch-one GEMVs) pinned bit for bit: against the committed
fixtures generated from the reference's own sources (tests/golden/make_golden_core.py) and, where a reference
checkout was available at build time, against oracle/_ref directly on fresh random inputs."""
import ctypes as C
import importlib.util
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests import fixtures as fx

HERE = os.path.dirname(os.path.abspath(__file__))
u16p, u8p, f32p = C.POINTER(C.c_uint16), C.POINTER(C.c_uint8), C.POINTER(C.c_float)


def p(a, ty=u16p):
    return a.ctypes.data_as(ty)


def generator():
    spec = importlib.util.spec_from_file_location("make_golden_core", os.path.join(HERE, "golden", "make_golden_core.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def gold():
    orc.build()
    return np.load(os.path.join(HERE, "golden", "reference_core_ops.npz"))


def same_f32(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def test_gdn_recurrence_against_the_golden_steps(gold):
    state = generator().structured_state()
    out, new_state = orc.gated_delta_net_update(gold["gdn_conv"], gold["gdn_a"], gold["gdn_b"], gold["gdn_A_log"],
                                                gold["gdn_dt_bias"], state, 1e-6)
    assert np.array_equal(out, gold["gdn_out_want"])
    assert np.array_equal(new_state[gold["gdn_state_heads"]], gold["gdn_state_want"])


def test_softmax_gqa_and_gemvs_against_golden(gold):
    assert same_f32(orc.softmax(gold["softmax_x"]), gold["softmax_want"])
    out, probs = orc.gqa_attention(gold["gqa_q"], gold["gqa_k"], gold["gqa_v"], 0.0625)
    assert np.array_equal(out, gold["gqa_out_want"]) and same_f32(probs, gold["gqa_probs_want"])
    assert same_f32(orc.bf16_gemv(gold["gemv_w"], gold["gemv_x"]), gold["gemv_want"])
    assert same_f32(orc.nvfp4_gemv(gold["nvfp4_gemv_packed"], gold["nvfp4_gemv_scales"], float(gold["nvfp4_gemv_scale2"][0]),
                                   gold["gemv_x"]), gold["nvfp4_gemv_want"])


def test_greedy_argmax_rule():
    enc = orc.bf16_encode
    v = enc(np.array([1.0, 3.5, -2.0, 3.5, 0.25], np.float32))
    assert orc.greedy_argmax(v) == (1, int(v[1]), 0)                      # earliest of equal maxima
    z = np.array([0x8000, 0x0000, 0x8000], np.uint16)
    assert orc.greedy_argmax(z) == (0, 0x8000, 0)                         # -0 == +0: the earlier index, its own bits
    n = np.array([0x7FC0, 0x7F80, 0xBF80, 0xFF80], np.uint16)             # NaN, +inf, -1, -inf
    assert orc.greedy_argmax(n) == (2, 0xBF80, 1)                         # non-finite skipped and flagged
    assert orc.greedy_argmax(np.array([0x7F80, 0xFFC0], np.uint16)) == (0xFFFFFFFF, 0, 1)
    assert orc.greedy_argmax(np.zeros(0, np.uint16)) == (0xFFFFFFFF, 0, 0)


@pytest.fixture(scope="module")
def ref():
    orc.build()
    r = orc.ref_lib()
    if r is None:
        pytest.skip("oracle/_ref not built (no reference checkout at build time)")
    return r


@pytest.mark.parametrize("seed,tokens", [(1, 1), (2, 2), (3, 5)])
def test_gdn_recurrence_equals_the_reference(ref, seed, tokens):
    rng = np.random.default_rng(seed)
    conv = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (tokens, 10240)), 0.0005) if seed == 3 else fx.normal_bf16(rng, (tokens, 10240))
    a, b = fx.normal_bf16(rng, (tokens, 48), 2.0), fx.normal_bf16(rng, (tokens, 48), 2.0)
    a[0, :4] = orc.bf16_encode(np.array([30.0, -30.0, 19.99, 20.01], np.float32))   # both softplus branches
    A_log = orc.bf16_encode(rng.uniform(-4.0, 1.5, 48).astype(np.float32))
    dt_bias = orc.bf16_encode(rng.uniform(-3.0, 3.0, 48).astype(np.float32))
    state = fx.normal_bf16(rng, (48, 128, 128), 0.05)
    got_out, got_state = orc.gated_delta_net_update(conv, a, b, A_log, dt_bias, state, 1e-6)
    st = state.copy()
    for t in range(tokens):
        o = np.empty(6144, np.uint16)
        assert ref.gdn_update(p(np.ascontiguousarray(conv[t])), p(np.ascontiguousarray(a[t])), p(np.ascontiguousarray(b[t])),
                              p(A_log), p(dt_bias), p(st), p(st), 1e-6, p(o)) == 0
        nan_g, nan_w = orc.bf16_is_nan(got_out[t]), orc.bf16_is_nan(o)
        assert np.array_equal(nan_g, nan_w) and np.array_equal(got_out[t][~nan_w], o[~nan_w]), f"step {t}"
    nan_w = orc.bf16_is_nan(st)
    assert np.array_equal(orc.bf16_is_nan(got_state), nan_w) and np.array_equal(got_state[~nan_w], st[~nan_w])


@pytest.mark.parametrize("length", [1, 2, 33, 257])
def test_gqa_attention_and_softmax_equal_the_reference(ref, length):
    rng = np.random.default_rng(length)
    q = fx.normal_bf16(rng, (24, 256))
    kc, vc = fx.normal_bf16(rng, (length, 4, 256)), fx.normal_bf16(rng, (length, 4, 256))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(256.0)))
    out, probs = orc.gqa_attention(q, kc, vc, scale)
    want_p = np.empty((24, length), np.float32)
    want = np.empty((24, 256), np.uint16)
    assert ref.gqa(p(q), p(kc), p(vc), 24, 4, length, 256, scale, p(want_p, f32p), want_p.size, p(want)) == 0
    assert np.array_equal(out, want) and same_f32(probs, want_p)
    x = (rng.standard_normal((7, length)) * 6).astype(np.float32)
    y = np.empty_like(x)
    assert ref.softmax(p(x, f32p), 7, length, p(y, f32p)) == 0
    assert same_f32(orc.softmax(x), y)
    # the gate epilogue is the sigmoid-gate op on the rounded attention output
    gate = fx.normal_bf16(rng, (24, 256), 2.0)
    gated, _ = orc.gqa_attention(q, kc, vc, scale, gate=gate)
    assert np.array_equal(gated, orc.sigmoid_gate(want, gate))


@pytest.mark.parametrize("rows,cols", [(3, 16), (17, 5120), (5, 17408)])
def test_gemvs_equal_the_reference(ref, rows, cols):
    rng = np.random.default_rng([rows, cols])
    w, x = fx.normal_bf16(rng, (rows, cols), 0.05), fx.normal_bf16(rng, (cols,))
    want = np.empty(rows, np.float32)
    assert ref.bf16_gemv(p(w), p(x), rows, cols, p(want, f32p)) == 0
    assert same_f32(orc.bf16_gemv(w, x), want)
    packed = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(0, 0x7F, size=(rows, cols // 16), dtype=np.uint8)
    assert ref.nvfp4_gemv(p(packed, u8p), p(scales, u8p), 0.004, p(x), rows, cols, p(want, f32p)) == 0
    assert same_f32(orc.nvfp4_gemv(packed, scales, 0.004, x), want)
