"""GPU parity tests of the operators BETWEEN the fused layer ops, through the C ABI, against the CPU oracle
(q3x_oracle_core.c, itself pinned to the reference's sources): the gated-delta-net recurrence (alone and with
the gated RMSNorm epilogue), batch-one GQA attention with the sigmoid output gate, row softmax and the greedy
argmax.

Tolerances: bf16 outputs within 1 bf16 ulp of the host op where a single FP32 result is rounded once
(attention output, first recurrence step); for the multi-token recurrence, whose bf16 state feeds back into
itself, the reference's own acceptance rule max(2e-3, 8e-3 |e|) as the hard bound plus a 1-ulp quota; FP32
outputs (softmax) within 1e-5 relative; argmax exact.
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


def gdn_case(rng, tokens, state_std=0.05):
    conv = fx.normal_bf16(rng, (tokens, 10240))
    a, b = fx.normal_bf16(rng, (tokens, 48), 2.0), fx.normal_bf16(rng, (tokens, 48), 2.0)
    a[0, :4] = orc.bf16_encode(np.array([30.0, -30.0, 19.99, 20.01], np.float32))  # both softplus branches
    A_log = orc.bf16_encode(rng.uniform(-4.0, 1.5, 48).astype(np.float32))
    dt_bias = orc.bf16_encode(rng.uniform(-3.0, 3.0, 48).astype(np.float32))
    state = fx.normal_bf16(rng, (48, 128, 128), state_std)
    return conv, a, b, A_log, dt_bias, state


@pytest.mark.parametrize("tokens", [1, 2, 7, 16, 40])
@pytest.mark.parametrize("in_place", [False, True])
def test_gdn_recurrence(g, tokens, in_place):
    rng = np.random.default_rng([tokens, int(in_place), 71])
    conv, a, b, A_log, dt_bias, state = gdn_case(rng, tokens)
    want_out, want_state = orc.gated_delta_net_update(conv, a, b, A_log, dt_bias, state, EPS)
    d_state = g.Dev(state)
    d_new = d_state if in_place else g.empty_like_dev(state.shape)
    out = g.empty_like_dev((tokens, 6144))
    g.capi.check("q3x_b200_gated_delta_net_update", g.Dev(conv), tokens, g.Dev(a), g.Dev(b), g.Dev(A_log),
                 g.Dev(dt_bias), d_state, d_new, EPS, out, None)
    g.sync()
    got_out, got_state = out.get(), d_new.get()
    assert out.guards_intact() and d_new.guards_intact()
    if not in_place:
        assert np.array_equal(d_state.get(), state), "the input state must stay untouched"
    # first step: one rounding after FP32 sums in another order
    g.assert_bf16_within(got_out[0], want_out[0], 1, 0.97, "output of the first step")
    g.assert_reference_tolerance(got_out, want_out, "outputs")
    # (the state feeds back into itself: after many steps a few elements per million drift two ulps)
    g.assert_reference_tolerance(got_state, want_state, "persisted state", amplified=tokens > 1)
    # an updated state element is a difference of two products, so where it cancels a rounding-level change of
    # the prediction is many ulps OF THE RESULT; the bound that holds is half an ulp of the operands' magnitude
    _, exact = g.ulp_report(got_state, want_state)
    assert exact > (0.999 if tokens == 1 else 0.99), exact
    a_, e_ = orc.bf16_decode(got_state).astype(np.float64), orc.bf16_decode(want_state).astype(np.float64)
    worst_abs, top = float(np.max(np.abs(a_ - e_))), float(np.max(np.abs(e_)))
    # (one step: half an ulp at the largest magnitude; many steps: the bf16 state feeds back, one to two ulps)
    assert worst_abs <= (2.0 ** -9 if tokens == 1 else 2.0 ** -7) * top, (worst_abs, top)
    _, exact_out = g.ulp_report(got_out, want_out)
    assert exact_out > 0.90, exact_out


def test_gdn_recurrence_is_the_same_token_by_token(g):
    """Carrying the state through memory between single-token calls gives the bytes of one multi-token call
    (the state crosses a bf16 boundary after every step either way)."""
    rng = np.random.default_rng(72)
    tokens = 9
    conv, a, b, A_log, dt_bias, state = gdn_case(rng, tokens)
    d_conv, d_a, d_b, d_A, d_dt = g.Dev(conv), g.Dev(a), g.Dev(b), g.Dev(A_log), g.Dev(dt_bias)
    s1, s2 = g.Dev(state), g.Dev(state)
    o1, o2 = g.empty_like_dev((tokens, 6144)), g.empty_like_dev((tokens, 6144))
    g.capi.check("q3x_b200_gated_delta_net_update", d_conv, tokens, d_a, d_b, d_A, d_dt, s1, s1, EPS, o1, None)
    for t in range(tokens):
        g.capi.check("q3x_b200_gated_delta_net_update", d_conv.ptr_at(t * 10240), 1, d_a.ptr_at(t * 48), d_b.ptr_at(t * 48),
                     d_A, d_dt, s2, s2, EPS, o2.ptr_at(t * 6144), None)
    g.sync()
    g.assert_bits_equal(o1.get(), o2.get(), "outputs")
    g.assert_bits_equal(s1.get(), s2.get(), "state")


@pytest.mark.parametrize("tokens", [1, 5])
def test_gdn_recurrence_with_gated_norm_epilogue(g, tokens):
    rng = np.random.default_rng([tokens, 73])
    conv, a, b, A_log, dt_bias, state = gdn_case(rng, tokens)
    z = fx.normal_bf16(rng, (tokens, 6144))
    w = orc.bf16_encode((0.75 + rng.random(128) * 0.5).astype(np.float32))
    d_in = [g.Dev(x) for x in (conv, a, b, A_log, dt_bias)]
    s1, s2 = g.Dev(state), g.Dev(state)
    raw, fused = g.empty_like_dev((tokens, 6144)), g.empty_like_dev((tokens, 6144))
    g.capi.check("q3x_b200_gated_delta_net_update", d_in[0], tokens, *d_in[1:], s1, s1, EPS, raw, None)
    g.capi.check("q3x_b200_gated_delta_net_update_rms_norm_silu_gate", d_in[0], tokens, *d_in[1:], s2, s2, EPS, g.Dev(w),
                 g.Dev(z), EPS, fused, None)
    g.sync()
    g.assert_bits_equal(s1.get(), s2.get(), "state with and without the epilogue")
    # the epilogue on the GPU's own rounded raw output: the gated-norm host op, within 1 ulp
    want = orc.rms_norm_rows(raw.get().reshape(tokens, 48, 128), w, EPS, centered=False,
                             gate=z.reshape(tokens, 48, 128)).reshape(tokens, 6144)
    g.assert_bf16_within(fused.get(), want, 1, 0.98, "recurrence + gated norm")
    # and the same bytes as the stand-alone gated-norm kernel on that raw output
    alone = g.empty_like_dev((tokens, 6144))
    g.capi.check("q3x_b200_rms_norm_silu_gate", raw, g.Dev(w), g.Dev(z), tokens * 48, 128, EPS, alone, None)
    g.sync()
    worst, exact = g.ulp_report(fused.get(), alone.get())
    assert worst <= 1 and exact > 0.99


def test_gdn_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x100000
    args = [fake, 1, fake + (1 << 26), fake + (2 << 26), fake + (3 << 26), fake + (4 << 26), fake + (5 << 26),
            fake + (6 << 26), EPS, fake + (7 << 26), None]
    bad_eps = list(args); bad_eps[8] = 0.0
    assert g.capi.call("q3x_b200_gated_delta_net_update", *bad_eps) == inv
    null_state = list(args); null_state[6] = None
    assert g.capi.call("q3x_b200_gated_delta_net_update", *null_state) == inv
    out_on_state = list(args); out_on_state[9] = args[7] + 64
    assert g.capi.call("q3x_b200_gated_delta_net_update", *out_on_state) == inv
    partial = list(args); partial[7] = args[6] + 256
    assert g.capi.call("q3x_b200_gated_delta_net_update", *partial) == inv
    empty = list(args); empty[1] = 0
    assert g.capi.call("q3x_b200_gated_delta_net_update", *empty) == 0


# ------------------------------------------------------------------------------------------ attention

@pytest.mark.parametrize("length", [1, 2, 7, 63, 64, 65, 129, 1000, 4097])
@pytest.mark.parametrize("gated", [True, False])
def test_gqa_decode(g, length, gated):
    rng = np.random.default_rng([length, int(gated), 81])
    q = fx.normal_bf16(rng, (24, 256))
    kc, vc = fx.normal_bf16(rng, (length, 4, 256)), fx.normal_bf16(rng, (length, 4, 256))
    gate = fx.normal_bf16(rng, (24, 256), 2.0)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(256.0)))
    words = g.capi.lib().q3x_b200_gqa_decode_workspace_floats(length)
    ws = g.empty_like_dev((words,), dtype=np.float32, fill=np.nan)  # stale contents must not matter
    out = g.empty_like_dev((24, 256))
    g.capi.check("q3x_b200_gqa_attention_decode_sigmoid_gate", g.Dev(q), g.Dev(kc), g.Dev(vc), length, scale, ws, words,
                 g.Dev(gate) if gated else None, out, None)
    g.sync()
    want, _ = orc.gqa_attention(q, kc, vc, scale, gate=gate if gated else None)
    assert out.guards_intact() and ws.guards_intact()
    # one rounding of an FP32 weighted average of values of magnitude ~1, summed in another order: 1 ulp plus
    # a rounding-level fraction of the terms' magnitude; the gate multiplies the ROUNDED attention, so a 1-ulp
    # difference there passes through (up to 3 ulps of the smaller gated value)
    g.assert_sum_within(out.get(), want, 3 if gated else 1, 1e-5, 0.99, "decode attention")
    g.assert_reference_tolerance(out.get(), want, "decode attention")


def test_gqa_decode_long_cache_and_rejections(g):
    """A cache long enough for every split to be busy (one CTA per SM and KV head), sharp scores so the running
    maximum moves, against the oracle on the full length."""
    rng = np.random.default_rng(82)
    length = 20000
    q = fx.normal_bf16(rng, (24, 256), 3.0)
    kc, vc = fx.normal_bf16(rng, (length, 4, 256)), fx.normal_bf16(rng, (length, 4, 256))
    gate = fx.normal_bf16(rng, (24, 256), 2.0)
    scale = 0.0625
    words = g.capi.lib().q3x_b200_gqa_decode_workspace_floats(length)
    ws = g.empty_like_dev((words,), dtype=np.float32)
    out = g.empty_like_dev((24, 256))
    d_q, d_k, d_v, d_g = g.Dev(q), g.Dev(kc), g.Dev(vc), g.Dev(gate)
    g.capi.check("q3x_b200_gqa_attention_decode_sigmoid_gate", d_q, d_k, d_v, length, scale, ws, words, d_g, out, None)
    g.sync()
    want, _ = orc.gqa_attention(q, kc, vc, scale, gate=gate)
    g.assert_sum_within(out.get(), want, 3, 1e-5, 0.99, "long-cache decode attention")
    inv = g.capi.CUDA_ERROR_INVALID_VALUE
    call = lambda *a: g.capi.call("q3x_b200_gqa_attention_decode_sigmoid_gate", *a)
    assert call(d_q, d_k, d_v, 0, scale, ws, words, d_g, out, None) == inv
    assert call(d_q, d_k, d_v, length, float("nan"), ws, words, d_g, out, None) == inv
    assert call(d_q, d_k, d_v, length, scale, ws, words - 1, d_g, out, None) == inv
    assert call(d_q, d_k, d_v, length, scale, ws, words, d_g, d_q, None) == inv        # out on the query
    assert call(d_q, d_k, d_v, length, scale, None, words, d_g, out, None) == inv


# ------------------------------------------------------------------------------------------ logits

@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 37), (24, 4097), (2, 248320)])
def test_softmax(g, rows, cols):
    rng = np.random.default_rng([rows, cols, 91])
    x = (rng.standard_normal((rows, cols)) * 5).astype(np.float32)
    x[0, 0] = 60.0
    if rows > 1:
        x[1, :] = -3.0e4
    d_x = g.Dev(x)
    out = g.empty_like_dev((rows, cols), dtype=np.float32)
    g.capi.check("q3x_b200_softmax", d_x, rows, cols, out, None)
    g.capi.check("q3x_b200_softmax", d_x, rows, cols, d_x, None)  # in place
    g.sync()
    want = orc.softmax(x).astype(np.float64)
    got = out.get().astype(np.float64)
    big = want > 1e-30
    assert np.max(np.abs(got[big] - want[big]) / want[big]) <= 1e-5
    assert np.all(np.abs(got[~big] - want[~big]) <= 1e-35)
    assert np.array_equal(out.get().view(np.uint32), d_x.get().view(np.uint32))
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("count", [1, 2, 255, 257, 5000, 248320])
def test_greedy_argmax(g, count):
    rng = np.random.default_rng([count, 92])
    x = fx.normal_bf16(rng, (count,), 3.0)
    if count > 300:
        top = np.sort(orc.bf16_decode(x))[-1]
        x[[count // 3, count // 2, count - 7]] = orc.bf16_encode(np.array([top], np.float32))[0]  # ties
        x[[5, count - 1]] = [0x7F80, 0xFFC0]                                                      # +inf, NaN
    ws = g.empty_like_dev((33 * 2,), dtype=np.uint32, fill=0xDEADBEEF)
    g.capi.check("q3x_b200_bf16_greedy_argmax", g.Dev(x), count, ws, None)
    g.sync()
    rec = ws.get()
    got = (int(rec[0]), int(rec[1] & 0xFFFF), int(rec[1] >> 16))
    assert got == orc.greedy_argmax(x)
    assert ws.guards_intact()


def test_greedy_argmax_special_vectors(g):
    cases = [np.array([0x8000, 0x0000, 0x8000], np.uint16), np.array([0x7FC0, 0x7F80, 0xBF80, 0xFF80], np.uint16),
             np.array([0x7F80, 0xFFC0], np.uint16), np.full(1000, 0xFF7F, np.uint16)]
    for x in cases:
        ws = g.empty_like_dev((66,), dtype=np.uint32)
        g.capi.check("q3x_b200_bf16_greedy_argmax", g.Dev(x), x.size, ws, None)
        g.sync()
        rec = ws.get()
        assert (int(rec[0]), int(rec[1] & 0xFFFF), int(rec[1] >> 16)) == orc.greedy_argmax(x)


# ------------------------------------------------------------------------------------------ batch-one projections

def gemv_tolerance(cols, want):
    """The reference's acceptance rule for a GEMV row (tests/reference_gemv_cuda_test.cu:36-45)."""
    return 5.0e-5 * np.sqrt(cols) + 5.0e-4 * np.abs(want)


@pytest.mark.parametrize("rows,cols", [(1, 16), (3, 32), (17, 5120), (130, 17408), (5120, 6144), (37, 1040)])
@pytest.mark.parametrize("misalign", [0, 1])
def test_gemvs(g, rows, cols, misalign):
    rng = np.random.default_rng([rows, cols, misalign, 95])
    x = fx.normal_bf16(rng, (cols,))
    d_x = g.Dev(x, misalign)
    # bf16 weights
    w = fx.normal_bf16(rng, (rows, cols), 0.05)
    o32, o16 = g.empty_like_dev((rows,), dtype=np.float32), g.empty_like_dev((rows,))
    g.capi.check("q3x_b200_bf16_gemv", g.Dev(w, misalign), d_x, rows, cols, o32, o16, None)
    g.sync()
    want = orc.bf16_gemv(w, x)
    assert np.all(np.abs(o32.get() - want) <= gemv_tolerance(cols, want)), "bf16 GEMV"
    g.assert_bits_equal(o16.get(), orc.bf16_encode(o32.get()), "bf16 output = rounding of the FP32 output")
    # norm-wise accuracy far inside the acceptance rule: 1e-5 of sum |w x|
    mag = np.abs(orc.bf16_decode(w).astype(np.float64)) @ np.abs(orc.bf16_decode(x).astype(np.float64))
    assert np.all(np.abs(o32.get() - want) <= 1e-5 * mag + 1e-30)
    # FP8 weights with a per-tensor scale
    w8 = rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
    w8[(w8 & 0x7F) == 0x7F] = 0x3C  # no NaN codes
    g.capi.check("q3x_b200_fp8_gemv", g.Dev(w8, misalign), 0.0123, d_x, rows, cols, o32, None, None)
    g.sync()
    L = orc.oracle_lib()
    e4 = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    wf = (e4[w8] * np.float32(0.0123)).astype(np.float32)
    want8 = (wf.astype(np.float64) @ orc.bf16_decode(x).astype(np.float64))
    mag8 = np.abs(wf.astype(np.float64)) @ np.abs(orc.bf16_decode(x).astype(np.float64))
    assert np.all(np.abs(o32.get() - want8) <= 2e-5 * mag8 + 1e-30), "FP8 GEMV"
    # NVFP4 weights
    if cols % 16 == 0:
        packed = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
        scales = rng.integers(0x18, 0x58, size=(rows, cols // 16), dtype=np.uint8)
        g.capi.check("q3x_b200_nvfp4_gemv", g.Dev(packed, misalign), g.Dev(scales, misalign), 0.004, d_x, rows, cols, o32,
                     o16, None)
        g.sync()
        want4 = orc.nvfp4_gemv(packed, scales, 0.004, x)
        assert np.all(np.abs(o32.get() - want4) <= gemv_tolerance(cols, want4)), "NVFP4 GEMV"
        deq = orc.nvfp4_dequantize(packed, scales, 0.004).astype(np.float64)
        mag4 = np.abs(deq) @ np.abs(orc.bf16_decode(x).astype(np.float64))
        assert np.all(np.abs(o32.get() - want4) <= 1e-5 * mag4 + 1e-30)
        g.assert_bits_equal(o16.get(), orc.bf16_encode(o32.get()), "NVFP4: bf16 output = rounding of the FP32 output")
    assert o32.guards_intact() and o16.guards_intact()


@pytest.mark.parametrize("rows,cols", [(40, 5120), (16, 192), (33, 17408)])
def test_gemvs_over_the_activation_range(g, rows, cols):
    """The narrow-weight GEMVs over the activation's range: very large, very small and widely spread activations
    keep the norm-wise accuracy, and non-finite activations give the oracle's non-finite results."""
    rng = np.random.default_rng([rows, cols, 98])
    packed = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(0x18, 0x58, size=(rows, cols // 16), dtype=np.uint8)
    w8 = rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
    w8[(w8 & 0x7F) == 0x7F] = 0x3C
    L = orc.oracle_lib()
    e4 = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    d_p, d_s, d_w8 = g.Dev(packed), g.Dev(scales), g.Dev(w8)
    o32 = g.empty_like_dev((rows,), dtype=np.float32)
    base = rng.standard_normal(cols).astype(np.float32)
    spread = base * np.exp2(rng.integers(-40, 1, size=cols)).astype(np.float32)
    for name, xf in (("huge", base * np.float32(1e30)), ("tiny", base * np.float32(1e-30)), ("spread", spread),
                     ("zero", np.zeros(cols, np.float32))):
        x = orc.bf16_encode(xf)
        xd = orc.bf16_decode(x).astype(np.float64)
        d_x = g.Dev(x)
        g.capi.check("q3x_b200_nvfp4_gemv", d_p, d_s, 0.004, d_x, rows, cols, o32, None, None)
        g.sync()
        deq = orc.nvfp4_dequantize(packed, scales, 0.004).astype(np.float64)
        assert np.all(np.abs(o32.get() - deq @ xd) <= 1e-5 * (np.abs(deq) @ np.abs(xd)) + 1e-37), f"NVFP4, {name} activation"
        g.capi.check("q3x_b200_fp8_gemv", d_w8, 0.0123, d_x, rows, cols, o32, None, None)
        g.sync()
        wf = (e4[w8] * np.float32(0.0123)).astype(np.float64)
        assert np.all(np.abs(o32.get() - wf @ xd) <= 2e-5 * (np.abs(wf) @ np.abs(xd)) + 1e-37), f"FP8, {name} activation"
    x = orc.bf16_encode(base)
    x[5], x[cols - 3] = 0x7F80, 0x7FC0  # +inf and a NaN
    g.capi.check("q3x_b200_nvfp4_gemv", d_p, d_s, 0.004, g.Dev(x), rows, cols, o32, None, None)
    g.sync()
    want = orc.nvfp4_gemv(packed, scales, 0.004, x)
    assert np.array_equal(np.isnan(o32.get()), np.isnan(want)) and np.all(np.isnan(want))
    x[cols - 3] = 0x3F80  # only the infinity is left: rows whose weight at column 5 is zero give NaN, the others +-inf
    g.capi.check("q3x_b200_nvfp4_gemv", d_p, d_s, 0.004, g.Dev(x), rows, cols, o32, None, None)
    g.sync()
    want = orc.nvfp4_gemv(packed, scales, 0.004, x)
    assert np.array_equal(np.isnan(o32.get()), np.isnan(want))
    assert np.array_equal(o32.get()[~np.isnan(want)], want[~np.isnan(want)])


def test_gemv_consumes_the_quantisers_layout(g):
    """Codes and block scales written by the library's own NVFP4 quantiser are the GEMV's weight layout: a
    matrix quantised row-wise by q3x_b200_nvfp4_quantize_dynamic and multiplied by a vector through
    q3x_b200_nvfp4_gemv equals the GEMV oracle on those bytes, and is close to the bf16 product."""
    rng = np.random.default_rng(96)
    rows, cols = 256, 5120
    w = fx.normal_bf16(rng, (rows, cols), 0.03)
    x = fx.normal_bf16(rng, (cols,))
    codes = g.empty_like_dev((rows, cols // 2), dtype=np.uint8)
    scales = g.empty_like_dev((rows, cols // 16), dtype=np.uint8)
    gs = g.empty_like_dev((1,), dtype=np.float32)
    g.capi.check("q3x_b200_nvfp4_quantize_dynamic", g.Dev(w), rows, cols, 0, g.scratch_for(rows, 0), gs, codes, scales, None)
    g.sync()
    scale_2 = float(gs.get()[0])
    out = g.empty_like_dev((rows,), dtype=np.float32)
    g.capi.check("q3x_b200_nvfp4_gemv", codes, scales, scale_2, g.Dev(x), rows, cols, out, None, None)
    g.sync()
    want = orc.nvfp4_gemv(codes.get(), scales.get(), scale_2, x)
    assert np.all(np.abs(out.get() - want) <= gemv_tolerance(cols, want))
    exact = orc.bf16_gemv(w, x)
    assert np.corrcoef(out.get(), exact)[0, 1] > 0.99  # 4-bit weights: close, not equal


def test_gemv_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x100000
    assert g.capi.call("q3x_b200_nvfp4_gemv", fake, fake + (1 << 28), 0.1, fake + (2 << 28), 4, 24, fake + (3 << 28), None, None) == inv
    assert g.capi.call("q3x_b200_nvfp4_gemv", fake, fake + (1 << 28), -1.0, fake + (2 << 28), 4, 32, fake + (3 << 28), None, None) == inv
    assert g.capi.call("q3x_b200_bf16_gemv", fake, fake + (2 << 28), 4, 32, None, None, None) == inv     # no output
    assert g.capi.call("q3x_b200_bf16_gemv", fake, fake + (2 << 28), 4, 32, fake + 8, None, None) == inv  # out on weights
    assert g.capi.call("q3x_b200_bf16_gemv", None, None, 0, 32, None, None, None) == 0


# ------------------------------------------------------------------------------------------ compact q / k conv

@pytest.mark.parametrize("tokens", [1, 63, 64, 65, 200, 513])
def test_causal_conv_compact_qk(g, tokens):
    """The conv with the compact q / k operands of the chunked GDN prefill: `out` is the plain conv output,
    compact_q / compact_k hold the L2-normalised heads in [chunk, head, 64, 128] order with a zeroed tail;
    everything is the bytes of the token-major entry points re-laid out."""
    rng = np.random.default_rng([tokens, 97])
    C_ = 10240
    raw = fx.normal_bf16(rng, (tokens, C_))
    w = fx.normal_bf16(rng, (C_, 4), 0.5)
    hist = fx.normal_bf16(rng, (C_, 3))
    qs = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    chunks = (tokens + 63) // 64
    d_raw, d_w = g.Dev(raw), g.Dev(w)
    h1, h2, h3 = g.Dev(hist), g.Dev(hist), g.Dev(hist)
    out, plain, fused = g.empty_like_dev((tokens, C_)), g.empty_like_dev((tokens, C_)), g.empty_like_dev((tokens, C_))
    cq = g.empty_like_dev((chunks, 16, 64, 128), fill=0x7777)
    ck = g.empty_like_dev((chunks, 16, 64, 128), fill=0x7777)
    g.capi.check("q3x_b200_causal_conv1d_silu_compact_qk", d_raw, tokens, d_w, h1, out, EPS, qs, cq, ck, None)
    g.capi.check("q3x_b200_causal_conv1d_silu", d_raw, tokens, C_, d_w, h2, plain, None)
    g.capi.check("q3x_b200_causal_conv1d_silu_l2norm", d_raw, tokens, d_w, h3, EPS, qs, fused, None)
    g.sync()
    g.assert_bits_equal(out.get(), plain.get(), "conv output of the compact form == plain conv")
    g.assert_bits_equal(h1.get(), h2.get(), "history")
    f = fused.get()
    want_q = np.zeros((chunks * 64, 16, 128), np.uint16)
    want_k = np.zeros((chunks * 64, 16, 128), np.uint16)
    want_q[:tokens] = f[:, :2048].reshape(tokens, 16, 128)
    want_k[:tokens] = f[:, 2048:4096].reshape(tokens, 16, 128)
    relayout = lambda a: a.reshape(chunks, 64, 16, 128).transpose(0, 2, 1, 3)
    g.assert_bits_equal(cq.get(), relayout(want_q), "compact q")
    g.assert_bits_equal(ck.get(), relayout(want_k), "compact k")
    assert cq.guards_intact() and ck.guards_intact() and out.guards_intact()
    # and against the oracle chain on the GPU's own conv output
    conv = plain.get()
    oq = orc.l2_normalize_heads(conv[:, :2048].reshape(-1, 128), EPS, qs).reshape(tokens, 16, 128)
    g.assert_bf16_within(cq.get().transpose(0, 2, 1, 3).reshape(-1, 16, 128)[:tokens], oq, 1, 0.98, "compact q vs oracle")
