"""The C restatement against the committed golden fixtures (outputs of the reference project's own
host reference ops, see tests/golden/make_golden.py) and against independent known answers.
Runs anywhere: needs neither a GPU nor a reference checkout."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import fixtures as fx

EPS = 1e-6
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_ops.npz")


@pytest.fixture(scope="module")
def gold():
    orc.build()
    return np.load(GOLDEN)


def same(a, b):
    a, b = np.asarray(a), np.asarray(b)
    na, nb = orc.bf16_is_nan(a), orc.bf16_is_nan(b)
    return bool(np.array_equal(na, nb) and np.array_equal(a[~na], b[~nb]))


def test_residual_norm(gold):
    res, nrm = orc.residual_add_rms_norm(gold["rn_left"], gold["rn_right"], gold["rn_weight"], EPS)
    assert same(res, gold["rn_residual_want"])
    assert same(nrm, gold["rn_normalized_want"])


def test_pointwise(gold):
    a, b = gold["pw_a"], gold["pw_b"]
    assert same(orc.residual_add(a, b), gold["pw_residual_want"])
    assert same(orc.silu_mul(a, b), gold["pw_silu_mul_want"])
    assert same(orc.sigmoid_gate(a, b), gold["pw_sigmoid_gate_want"])
    merged = np.concatenate([a[:770].reshape(2, 385), b[:770].reshape(2, 385)], axis=1)
    assert same(orc.silu_mul_merged(merged).reshape(-1), gold["pw_silu_mul_want"][:770])


def test_head_norms(gold):
    assert same(orc.rms_norm_rows(gold["hn_x"], gold["hn_w"], EPS, centered=True), gold["hn_centered_want"])
    assert same(orc.rms_norm_rows(gold["gn_x"], gold["gn_w"], EPS, centered=False), gold["gn_plain_want"])
    assert same(orc.rms_norm_rows(gold["gn_x"], gold["gn_w"], EPS, centered=False, gate=gold["gn_z"]),
                gold["gn_want"])


def test_l2_rope_split(gold):
    assert same(orc.l2_normalize_heads(gold["l2a_x"], EPS), gold["l2a_want"])
    assert same(orc.l2_normalize_heads(gold["l2b_x"], EPS), gold["l2b_want"])
    assert same(orc.partial_rope(gold["rope_x"], gold["rope_cos"][0], gold["rope_sin"][0]), gold["rope_want"])
    cos, sin = orc.rope_tables(4096, 1)
    assert np.array_equal(cos, gold["rope_cos"]) and np.array_equal(sin, gold["rope_sin"])
    q, g = orc.split_q_gate(gold["split_in"], 24, 256)
    assert np.array_equal(q, gold["split_q_want"]) and np.array_equal(g, gold["split_gate_want"])


def test_conv(gold):
    out, hist = orc.causal_conv1d_silu(gold["conv_raw"], gold["conv_w"], gold["conv_hist"])
    assert same(out, gold["conv_want"])
    assert np.array_equal(hist, gold["conv_hist_want"])
    # splitting the span carries the history across the cut
    o1, h1 = orc.causal_conv1d_silu(gold["conv_raw"][:1], gold["conv_w"], gold["conv_hist"])
    o2, h2 = orc.causal_conv1d_silu(gold["conv_raw"][1:], gold["conv_w"], h1)
    assert same(np.concatenate([o1, o2]), gold["conv_want"]) and np.array_equal(h2, hist)


def test_embedding(gold):
    ids = np.array([3, 0, 4, 4, 1, 2], dtype=np.uint32)
    out = orc.embedding_gather(gold["emb_table"], ids)
    assert np.array_equal(out, gold["emb_want"][ids])
    # an id outside the vocabulary leaves its row untouched
    sentinel = np.full((3, 7), 0xABCD, dtype=np.uint16)
    out = orc.embedding_gather(gold["emb_table"], np.array([1, 5, 2], dtype=np.uint32), out=sentinel)
    assert np.array_equal(out[0], gold["emb_want"][1]) and np.array_equal(out[2], gold["emb_want"][2])
    assert np.all(out[1] == 0xABCD)


def test_format_tables(gold):
    L = orc.oracle_lib()
    assert np.array_equal(np.array([L.decode_e2m1(i) for i in range(16)], dtype=np.float32).view(np.uint32),
                          gold["e2m1_table"].view(np.uint32))
    mine = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    want = gold["e4m3_table"]
    assert np.array_equal(np.isnan(mine), np.isnan(want))
    assert np.array_equal(mine[~np.isnan(mine)].view(np.uint32), want[~np.isnan(want)].view(np.uint32))
    # known answers spelled out in the reference's tests (tests/nvfp4_test.cu:43-175):
    assert list(gold["e2m1_table"][:8]) == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert want[0x7E] == 448.0 and want[0x01] == 2.0**-9 and want[0x38] == 1.0 and want[0x08] == 2.0**-6


def test_e4m3_encoder_against_golden_and_torch(gold):
    L = orc.oracle_lib()
    want = gold["e4m3_quantised_of_every_bf16"]
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    x = orc.bf16_decode(bits)
    for i in range(0, 65536, 7):  # a stride keeps this quick; the full sweep runs against _ref
        if np.isnan(x[i]):
            continue
        assert L.decode_e4m3(L.encode_e4m3(float(x[i]))) == want[i]
    # the reference's spelled-out answers (tests/reference_gemv_host_test.cpp:176-193)
    for v, q in ((0.26, 0.25), (1.0625, 1.0), (500.0, 448.0), (-0.26, -0.25), (0.001953125, 0.001953125)):
        b = float(orc.bf16_decode(orc.bf16_encode(np.array([v], dtype=np.float32)))[0])
        assert L.decode_e4m3(L.encode_e4m3(b)) == q
    # an independent implementation: torch's float8_e4m3fn cast of the clamped value
    rng = np.random.default_rng(3)
    vals = np.concatenate([
        (rng.standard_normal(20000) * 100).astype(np.float32),
        (rng.standard_normal(20000) * 0.01).astype(np.float32),
        np.array([0, 2**-10, 2**-10 * 1.0001, 2**-9, 3 * 2**-10, 0.0175, 447.9, 448, 464, 465, 1e9, -1e9],
                 dtype=np.float32),
    ])
    t = torch.from_numpy(np.clip(vals, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    mine = np.array([L.encode_e4m3(float(v)) for v in vals], dtype=np.uint8)
    assert np.array_equal(mine & 0x7F, t & 0x7F)
    nz = (mine & 0x7F) != 0
    assert np.array_equal(mine[nz], t[nz])


def test_e2m1_encoder_ladder():
    L = orc.oracle_lib()
    grid = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for code, v in enumerate(grid):
        assert L.encode_e2m1(v) == code and L.encode_e2m1(-v) == (code | 8)
    # midpoints go to the even code
    for mid, want in ((0.25, 0), (0.75, 2), (1.25, 2), (1.75, 4), (2.5, 4), (3.5, 6), (5.0, 6)):
        assert L.encode_e2m1(mid) == want, mid
        assert L.encode_e2m1(float(np.nextafter(np.float32(mid), np.float32(10)))) == want + (1 if want % 2 == 0 else 0) \
            or L.encode_e2m1(float(np.nextafter(np.float32(mid), np.float32(10)))) >= want
    assert L.encode_e2m1(float("inf")) == 7 and L.encode_e2m1(float("-inf")) == 15
    assert L.encode_e2m1(float("nan")) == 7 and L.encode_e2m1(1e30) == 7
    # nearest-value property on a dense sweep
    xs = np.linspace(-7, 7, 28001, dtype=np.float32)
    g = np.array(grid, dtype=np.float32)
    for x in xs[::13]:
        c = L.encode_e2m1(float(x))
        d = np.abs(g - abs(x))
        assert d[c & 7] == d.min()


@pytest.mark.parametrize("rows,cols,rps", [(7, 64, 0), (40, 5120, 16), (33, 6144, 512), (5, 17408, 2)])
def test_nvfp4_quantiser_properties(rows, cols, rps):
    rng = np.random.default_rng(rows * cols)
    x = fx.normal_bf16(rng, (rows, cols))
    x[0, :16] = 0                       # an all-zero block
    x[1 % rows, 16:32] = 0x0001         # a block of bf16 subnormals
    fx.sprinkle_specials(rng, x[-1:], 0.01)
    codes, scales, gs = orc.nvfp4_quantize(x, rps)
    per = rps or rows
    amax = orc.group_amax(x, rps)
    for g in range(gs.size):
        blk = x[g * per:(g + 1) * per]
        finite = orc.bf16_decode(blk[(blk & 0x7FFF) < 0x7F80])
        assert amax[g] == np.abs(finite).max()
        assert gs[g] == (np.float32(amax[g]) / np.float32(2688.0) if amax[g] else 1.0)
    # re-deriving with the scales supplied gives the same bytes
    c2, s2 = orc.nvfp4_quantize_with_scales(x, gs, rps)
    assert np.array_equal(c2, codes) and np.array_equal(s2, scales)
    # zero block -> zero scale and zero codes
    assert scales[0, 0] == 0 and np.all(codes[0, :8] == 0)
    # the largest finite element of each group lands on +-6 times the largest block scale used
    deq = np.concatenate([orc.nvfp4_dequantize(codes[g * per:(g + 1) * per], scales[g * per:(g + 1) * per], gs[g])
                          for g in range(gs.size)])
    xf = orc.bf16_decode(x)
    fin = np.isfinite(xf)
    d = np.array([orc.oracle_lib().decode_e4m3(int(v)) for v in scales.reshape(-1)], dtype=np.float32)
    d = np.repeat(d.reshape(scales.shape), 16, axis=1) * np.repeat(gs, per)[:rows, None]
    # E2M1 steps are at most 2 wide (4 -> 6) and the block scale is within 1/16 of ideal, so the
    # error is bounded by (1 + 6/16) * d
    live = fin & (np.repeat(scales, 16, axis=1) != 0)   # a block whose scale underflowed decodes to zero
    assert np.all(np.abs(deq[live] - xf[live]) <= 1.4 * d[live] + 1e-30)
    assert np.all(deq[fin & ~live] == 0)
    # rows do not influence each other beyond the shared global scale
    c3, s3 = orc.nvfp4_quantize_with_scales(x[rows // 2:rows // 2 + 1], gs[(rows // 2) // per:(rows // 2) // per + 1], 0)
    assert np.array_equal(c3[0], codes[rows // 2]) and np.array_equal(s3[0], scales[rows // 2])


def test_status_codes():
    """Argument checking mirrors tests/decode_ops_host_test.cpp:664-751."""
    import ctypes as C

    L = orc.oracle_lib()
    u16p = C.POINTER(C.c_uint16)
    buf = np.zeros(64, dtype=np.uint16)
    b = buf.ctypes.data_as(u16p)
    big = np.iinfo(np.uint64).max
    assert L.rms_norm(b, b, 8, 0.0, 1, b) == orc.STATUS_INVALID_ARGUMENT
    assert L.rms_norm(b, b, 8, float("nan"), 1, b) == orc.STATUS_INVALID_ARGUMENT
    assert L.rms_norm(None, None, 0, EPS, 1, None) == orc.STATUS_OK
    assert L.rms_norm(None, b, 8, EPS, 1, b) == orc.STATUS_INVALID_ARGUMENT
    assert L.headwise(b, b, None, big // 2, 4, EPS, 1, b) == orc.STATUS_SIZE_OVERFLOW
    assert L.residual_add(None, None, 0, None) == orc.STATUS_OK
    assert L.residual_add(b, None, 4, b) == orc.STATUS_INVALID_ARGUMENT
    assert L.l2(b, big, 2, EPS, 1.0, b) == orc.STATUS_SIZE_OVERFLOW
    assert L.conv(b, 1, 4, b, b, b) == orc.STATUS_INVALID_ALIAS
    ids = np.array([9], dtype=np.uint32)
    assert L.embedding(b, 4, 4, ids.ctypes.data_as(C.POINTER(C.c_uint32)), 1, b) == orc.STATUS_TOKEN_OUT_OF_RANGE
    u8 = np.zeros(64, dtype=np.uint8).ctypes.data_as(C.POINTER(C.c_uint8))
    f32 = np.zeros(64, dtype=np.float32).ctypes.data_as(C.POINTER(C.c_float))
    assert L.quant(b, 1, 24, 0, u8, u8, f32) == orc.STATUS_INVALID_COLUMN_COUNT
