"""GPU parity tests of the NVFP4 activation quantiser.  The requirement is bit-exact codes, E4M3
block scales and FP32 global scales given identical pre-quantisation values, so every comparison
feeds the CPU encoder the very bf16 tensor the GPU quantised."""
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


def sweep_values():
    rng = np.random.default_rng(31)
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    near = np.concatenate([np.nextafter(mids, np.float32(0)), mids, np.nextafter(mids, np.float32(9))])
    e4 = np.array([orc.oracle_lib().decode_e4m3(c) for c in range(0x7F)], dtype=np.float32)
    e4_mid = (e4[:-1] + e4[1:]) / np.float32(2)
    e4_near = np.concatenate([e4, e4_mid, np.nextafter(e4_mid, np.float32(0)), np.nextafter(e4_mid, np.float32(1e9))])
    vals = np.concatenate([
        near, -near, e4_near, -e4_near,
        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 6.0, 6.5, 447.0, 448.0, 449.0, 464.0, 480.0,
                  1e30, -1e30, 2.0**-10, 2.0**-9, 1.5 * 2.0**-10, 0.0009765626], dtype=np.float32),
        (rng.standard_normal(200_000) * 3).astype(np.float32),
        (rng.standard_normal(100_000) * 200).astype(np.float32),
        (rng.standard_normal(100_000) * 0.01).astype(np.float32),
        rng.integers(0, 2**32, size=100_000, dtype=np.uint64).astype(np.uint32).view(np.float32),
    ])
    return vals.astype(np.float32)


@pytest.mark.parametrize("fmt,name", [(0, "e4m3"), (1, "e2m1")])
def test_narrow_conversions_match_the_cpu_definition(g, fmt, name):
    """The hardware conversions the kernels use against the oracle's encoders on a sweep that holds
    every grid point, every midpoint and its neighbours, specials and random bit patterns."""
    vals = sweep_values()
    d = g.Dev(vals)
    out = g.empty_like_dev((vals.size,), dtype=np.uint8)
    g.capi.check("q3x_b200_debug_encode", d, vals.size, fmt, out, None)
    g.sync()
    L = orc.oracle_lib()
    enc = L.encode_e4m3 if fmt == 0 else L.encode_e2m1
    want = np.array([enc(float(v)) for v in vals], dtype=np.uint8)
    got = out.get()
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, [(float(vals[i]), hex(got[i]), hex(want[i])) for i in bad[:10]]


CASES = [(7, 64, 0), (40, 5120, 16), (33, 6144, 512), (5, 17408, 2), (512, 5120, 512), (513, 5120, 512), (1, 16, 0)]


def make_input(rows, cols, seed):
    rng = np.random.default_rng([rows, cols, seed])
    x = fx.normal_bf16(rng, (rows, cols))
    x[0, :16] = 0
    x[rows // 2, 16:32] = 0x0001
    if rows > 4:
        fx.sprinkle_specials(rng, x[-1:], 0.01)
    return x


@pytest.mark.parametrize("rows,cols,rps", CASES)
@pytest.mark.parametrize("misalign", [0, 1])
def test_quantize_dynamic(g, rows, cols, rps, misalign):
    x = make_input(rows, cols, 1)
    groups = 1 if rps == 0 else (rows + rps - 1) // rps
    dx = g.Dev(x, misalign)
    amax = g.scratch_for(rows, rps)
    gs = g.empty_like_dev((groups,), dtype=np.float32)
    codes = g.empty_like_dev((rows, cols // 2), dtype=np.uint8, misalign=misalign)
    scales = g.empty_like_dev((rows, cols // 16), dtype=np.uint8)
    g.capi.check("q3x_b200_nvfp4_quantize_dynamic", dx, rows, cols, rps, amax, gs, codes, scales, None)
    g.sync()
    want_c, want_s, want_g = orc.nvfp4_quantize(x, rps)
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32)), "global scales"
    g.assert_scratch_clean(amax, "quantize_dynamic")
    g.assert_bits_equal(scales.get(), want_s, "E4M3 block scales")
    g.assert_bits_equal(codes.get(), want_c, "E2M1 codes")
    assert codes.guards_intact() and scales.guards_intact() and gs.guards_intact() and amax.guards_intact()
    # the pieces, called one by one, give the same bytes
    amax2 = g.empty_like_dev((groups,), dtype=np.uint32, fill=77)  # an output here: the call zeroes it itself
    gs2 = g.empty_like_dev((groups,), dtype=np.float32)
    c2 = g.empty_like_dev((rows, cols // 2), dtype=np.uint8)
    s2 = g.empty_like_dev((rows, cols // 16), dtype=np.uint8)
    assert g.capi.lib().q3x_b200_nvfp4_group_count(rows, rps) == groups
    g.capi.check("q3x_b200_group_amax", dx, rows, cols, rps, amax2, None)
    g.capi.check("q3x_b200_amax_to_global_scale", amax2, groups, gs2, None)
    g.capi.check("q3x_b200_nvfp4_quantize", dx, rows, cols, rps, gs2, c2, s2, None)
    g.sync()
    assert np.array_equal(amax2.get() << 16, orc.group_amax(x, rps).view(np.uint32)), "group amax bits"
    g.assert_bits_equal(c2.get(), want_c, "codes (stepwise)")
    g.assert_bits_equal(s2.get(), want_s, "scales (stepwise)")


def test_quantize_round_trip_and_static_scale(g):
    """dequantise(GPU codes) reproduces E2M1 * E4M3 * global exactly, the formula of the reference's
    decoder (src/quantization/nvfp4.cpp:52-59); a caller-supplied (static) scale is honoured."""
    x = make_input(64, 5120, 2)
    gs = np.array([0.004, 0.0015], dtype=np.float32)
    dx, dg = g.Dev(x), g.Dev(gs)
    codes = g.empty_like_dev((64, 2560), dtype=np.uint8)
    scales = g.empty_like_dev((64, 320), dtype=np.uint8)
    g.capi.check("q3x_b200_nvfp4_quantize", dx, 64, 5120, 32, dg, codes, scales, None)
    g.sync()
    want_c, want_s = orc.nvfp4_quantize_with_scales(x, gs, 32)
    g.assert_bits_equal(codes.get(), want_c, "codes, static scale")
    g.assert_bits_equal(scales.get(), want_s, "scales, static scale")
    deq = orc.nvfp4_dequantize(codes.get()[:32], scales.get()[:32], gs[0])
    L = orc.oracle_lib()
    e2 = np.array([L.decode_e2m1(i) for i in range(16)], dtype=np.float32)
    e4 = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    c = codes.get()[:32]
    nib = np.stack([c & 0xF, c >> 4], axis=-1).reshape(32, 5120)
    manual = e2[nib] * np.repeat(e4[scales.get()[:32]], 16, axis=1) * gs[0]
    assert np.array_equal(deq.view(np.uint32), manual.astype(np.float32).view(np.uint32))


@pytest.mark.parametrize("tokens,rps", [(1, 0), (2, 0), (2, 1), (7, 0), (7, 512), (33, 16), (512, 512), (513, 512), (1024, 512), (2048, 512),
                                        (5000, 512), (8200, 512), (4096, 64), (1500, 0), (3000, 0), (6000, 0)])
@pytest.mark.parametrize("single_pass", [False, True])
def test_residual_norm_nvfp4(g, tokens, rps, single_pass):
    hidden = 5120
    entry = "q3x_b200_residual_add_rms_norm_nvfp4" + ("_single_pass" if single_pass else "")
    rng = np.random.default_rng([tokens, rps, 3])
    left, right = fx.normal_bf16(rng, (tokens, hidden)), fx.normal_bf16(rng, (tokens, hidden))
    w = fx.normal_bf16(rng, (hidden,), 0.02)
    groups = 1 if rps == 0 else (tokens + rps - 1) // rps
    dl, dr, dw = g.Dev(left), g.Dev(right), g.Dev(w)
    res, nrm = g.empty_like_dev((tokens, hidden)), g.empty_like_dev((tokens, hidden))
    amax = g.scratch_for(tokens, rps, fill=123456)
    gs = g.empty_like_dev((groups,), dtype=np.float32)
    codes = g.empty_like_dev((tokens, hidden // 2), dtype=np.uint8)
    scales = g.empty_like_dev((tokens, hidden // 16), dtype=np.uint8)
    st = g.capi.call(entry, dl, dr, dw, tokens, hidden, EPS, rps, res, nrm, amax, gs, codes, scales, None)
    if single_pass and st == g.capi.CUDA_ERROR_NOT_SUPPORTED:
        assert rps == 0 and tokens > 3000, "only a scale group too long to wait in L2 may be refused"
        pytest.skip("scale group too long for the single-kernel form")
    assert st == 0
    g.sync()
    g.assert_scratch_clean(amax, entry)
    want_r, want_n = orc.residual_add_rms_norm(left, right, w, EPS)
    g.assert_bits_equal(res.get(), want_r, "residual")
    g.assert_bf16_within(nrm.get(), want_n, 1, 0.98, "normalized")
    # identical pre-quantisation values -> identical bytes
    want_c, want_s, want_g = orc.nvfp4_quantize(nrm.get(), rps)
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32)), "global scale"
    g.assert_bits_equal(scales.get(), want_s, "block scales")
    g.assert_bits_equal(codes.get(), want_c, "codes")
    # and the un-fused sequence of entry points produces the same bytes
    r2, n2 = g.empty_like_dev((tokens, hidden)), g.empty_like_dev((tokens, hidden))
    c2 = g.empty_like_dev((tokens, hidden // 2), dtype=np.uint8)
    s2 = g.empty_like_dev((tokens, hidden // 16), dtype=np.uint8)
    g.capi.check("q3x_b200_residual_add_rms_norm", dl, dr, dw, tokens, hidden, EPS, r2, n2, None)
    g.capi.check("q3x_b200_nvfp4_quantize_dynamic", n2, tokens, hidden, rps, amax, gs, c2, s2, None)
    g.sync()
    g.assert_bits_equal(n2.get(), nrm.get(), "normalized, fused vs unfused")
    g.assert_bits_equal(c2.get(), codes.get(), "codes, fused vs unfused")
    g.assert_bits_equal(s2.get(), scales.get(), "scales, fused vs unfused")
    for d in (res, nrm, codes, scales, gs, amax):
        assert d.guards_intact()


@pytest.mark.parametrize("tokens,rps", [(1, 0), (2, 512), (2, 1), (9, 4), (512, 512), (600, 512), (2048, 512), (4608, 512), (9001, 512),
                                        (4100, 96), (1300, 0), (4000, 0)])
@pytest.mark.parametrize("single_pass", [False, True])
def test_gated_norm_nvfp4(g, tokens, rps, single_pass):
    heads, dim = 48, 128
    entry = "q3x_b200_rms_norm_silu_gate_nvfp4" + ("_single_pass" if single_pass else "")
    rng = np.random.default_rng([tokens, rps, 4])
    x, z = fx.normal_bf16(rng, (tokens, heads, dim)), fx.normal_bf16(rng, (tokens, heads, dim))
    w = orc.bf16_encode((0.75 + rng.random(dim) * 0.5).astype(np.float32))
    groups = 1 if rps == 0 else (tokens + rps - 1) // rps
    dx, dz, dw = g.Dev(x), g.Dev(z), g.Dev(w)
    out = g.empty_like_dev((tokens, heads * dim))
    amax = g.scratch_for(tokens, rps, fill=99)
    gs = g.empty_like_dev((groups,), dtype=np.float32)
    codes = g.empty_like_dev((tokens, heads * dim // 2), dtype=np.uint8)
    scales = g.empty_like_dev((tokens, heads * dim // 16), dtype=np.uint8)
    st = g.capi.call(entry, dx, dw, dz, tokens, heads, dim, EPS, rps, out, amax, gs, codes, scales, None)
    if single_pass and st == g.capi.CUDA_ERROR_NOT_SUPPORTED:
        assert rps == 0 and tokens > 3000, "only a scale group too long to wait in L2 may be refused"
        pytest.skip("scale group too long for the single-kernel form")
    assert st == 0
    g.sync()
    g.assert_scratch_clean(amax, entry)
    want = orc.rms_norm_rows(x, w, EPS, centered=False, gate=z).reshape(tokens, heads * dim)
    g.assert_bf16_within(out.get(), want, 1, 0.98, "gated norm")
    want_c, want_s, want_g = orc.nvfp4_quantize(out.get(), rps)
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32))
    g.assert_bits_equal(scales.get(), want_s, "block scales")
    g.assert_bits_equal(codes.get(), want_c, "codes")


@pytest.mark.parametrize("tokens,inter,rps", [(1, 17408, 512), (3, 17408, 0), (64, 17408, 512), (512, 17408, 512),
                                              (600, 17408, 512), (1030, 17408, 512), (40, 4096, 8), (33, 1040, 16),
                                              (2000, 17408, 0), (96, 512, 32)])
def test_silu_mul_nvfp4(g, tokens, inter, rps):
    rng = np.random.default_rng([tokens, inter, rps, 5])
    gate, up = fx.normal_bf16(rng, (tokens, inter)), fx.normal_bf16(rng, (tokens, inter))
    if tokens >= 33:
        fx.sprinkle_specials(rng, gate[-2:], 0.002)
    groups = 1 if rps == 0 else (tokens + rps - 1) // rps
    dg, du = g.Dev(gate), g.Dev(up)
    out = g.empty_like_dev((tokens, inter))
    scratch = g.scratch_for(tokens, rps, fill=0x13572468)
    gs = g.empty_like_dev((groups,), dtype=np.float32)
    codes = g.empty_like_dev((tokens, inter // 2), dtype=np.uint8)
    scales = g.empty_like_dev((tokens, inter // 16), dtype=np.uint8)
    g.capi.check("q3x_b200_silu_mul_nvfp4", dg, du, tokens, inter, rps, out, scratch, gs, codes, scales, None)
    g.sync()
    g.assert_scratch_clean(scratch, "pointwise + NVFP4")
    got = out.get()
    g.assert_bf16_within(got, orc.silu_mul(gate, up), 1, 0.98, "SwiGLU")
    # the same bytes as the stand-alone SwiGLU entry, and codes / scales derived from them bit for bit
    plain = g.empty_like_dev((tokens, inter))
    g.capi.check("q3x_b200_silu_mul", dg, du, tokens * inter, plain, None)
    g.sync()
    g.assert_bits_equal(got, plain.get(), "fused SwiGLU == stand-alone SwiGLU")
    want_c, want_s, want_g = orc.nvfp4_quantize(got, rps)
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32)), "global scales"
    g.assert_bits_equal(scales.get(), want_s, "block scales")
    g.assert_bits_equal(codes.get(), want_c, "codes")
    for d in (out, codes, scales, gs, scratch):
        assert d.guards_intact()
    assert np.array_equal(dg.get(), gate) and np.array_equal(du.get(), up)


def test_silu_mul_nvfp4_in_place_and_rejections(g):
    rng = np.random.default_rng(77)
    tokens, inter = 520, 17408
    gate, up = fx.normal_bf16(rng, (tokens, inter)), fx.normal_bf16(rng, (tokens, inter))
    dg, du = g.Dev(gate), g.Dev(up)
    scratch = g.scratch_for(tokens, 512)
    gs = g.empty_like_dev((2,), dtype=np.float32)
    codes = g.empty_like_dev((tokens, inter // 2), dtype=np.uint8)
    scales = g.empty_like_dev((tokens, inter // 16), dtype=np.uint8)
    g.capi.check("q3x_b200_silu_mul_nvfp4", dg, du, tokens, inter, 512, dg, scratch, gs, codes, scales, None)  # out == gate
    g.sync()
    got = dg.get()
    g.assert_bf16_within(got, orc.silu_mul(gate, up), 1, 0.98, "in-place SwiGLU")
    want_c, want_s, want_g = orc.nvfp4_quantize(got, 512)
    g.assert_bits_equal(codes.get(), want_c, "codes")
    g.assert_bits_equal(scales.get(), want_s, "scales")
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32))
    # host-visible argument errors are refused before anything is enqueued
    inv = g.capi.CUDA_ERROR_INVALID_VALUE
    assert g.capi.call("q3x_b200_silu_mul_nvfp4", dg, du, tokens, 17400, 512, dg, scratch, gs, codes, scales, None) == inv
    assert g.capi.call("q3x_b200_silu_mul_nvfp4", dg, du, tokens, inter, 512, dg.ptr_at(8), scratch, gs, codes, scales,
                       None) == inv
    assert g.capi.call("q3x_b200_silu_mul_nvfp4", dg, du, tokens, inter, 512, None, scratch, gs, codes, scales, None) == inv
    assert g.capi.call("q3x_b200_silu_mul_nvfp4", None, None, 0, inter, 512, None, None, None, None, None, None) == 0


def test_single_kernel_path_matches_two_kernel_path_over_many_launches(g):
    """The single-kernel form orders its two phases with device-side counters; the two-kernel form
    (reached through the entry with built-in scratch) uses stream order.  Same bytes, every time."""
    import torch

    T, H = 16384, 5120
    gen = torch.Generator(device="cuda").manual_seed(2024)
    bf = dict(device="cuda", dtype=torch.bfloat16)
    words = g.capi.lib().q3x_b200_nvfp4_scratch_words(T, 512)
    scratch = torch.zeros((words,), device="cuda", dtype=torch.int32)
    w = (torch.randn((H,), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    outs = []
    for _ in range(2):
        outs.append(dict(res=torch.empty((T, H), **bf), nrm=torch.empty((T, H), **bf),
                         gs=torch.empty(32, device="cuda", dtype=torch.float32),
                         codes=torch.empty((T, H // 2), device="cuda", dtype=torch.uint8),
                         scales=torch.empty((T, H // 16), device="cuda", dtype=torch.uint8)))
    for it in range(24):
        if it % 4 == 0:
            left = (torch.randn((T, H), generator=gen, device="cuda") * (1.0 + it)).to(torch.bfloat16)
            right = torch.randn((T, H), generator=gen, device="cuda").to(torch.bfloat16)
        a, b = outs
        g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4", left, right, w, T, H, EPS, 512, a["res"], a["nrm"], scratch,
                     a["gs"], a["codes"], a["scales"], None)
        g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4_static_scratch", left, right, w, T, H, EPS, 512, b["res"],
                     b["nrm"], b["gs"], b["codes"], b["scales"], None)
        g.sync()
        assert not bool(scratch.any().item()), f"launch {it}: scratch not left zero (or a bounded wait gave up)"
        for name in a:
            assert torch.equal(a[name].view(torch.uint8), b[name].view(torch.uint8)), f"launch {it}: {name} differs"


@pytest.mark.parametrize("tokens,width,rps", [(1, 6144, 512), (5, 6144, 0), (512, 6144, 512), (700, 6144, 512),
                                              (64, 1024, 16), (33, 1040, 16), (3000, 6144, 0)])
def test_sigmoid_gate_nvfp4(g, tokens, width, rps):
    rng = np.random.default_rng([tokens, width, rps, 6])
    value, gate = fx.normal_bf16(rng, (tokens, width)), fx.normal_bf16(rng, (tokens, width), 3.0)
    if tokens >= 33:
        fx.sprinkle_specials(rng, gate[-2:], 0.002)
    groups = 1 if rps == 0 else (tokens + rps - 1) // rps
    dv, dg = g.Dev(value), g.Dev(gate)
    out = g.empty_like_dev((tokens, width))
    scratch = g.scratch_for(tokens, rps, fill=0x0BADF00D)
    gs = g.empty_like_dev((groups,), dtype=np.float32)
    codes = g.empty_like_dev((tokens, width // 2), dtype=np.uint8)
    scales = g.empty_like_dev((tokens, width // 16), dtype=np.uint8)
    g.capi.check("q3x_b200_sigmoid_gate_nvfp4", dv, dg, tokens, width, rps, out, scratch, gs, codes, scales, None)
    g.sync()
    g.assert_scratch_clean(scratch, "pointwise + NVFP4")
    got = out.get()
    g.assert_bf16_within(got, orc.sigmoid_gate(value, gate), 1, 0.98, "sigmoid gate")
    plain = g.empty_like_dev((tokens, width))
    g.capi.check("q3x_b200_sigmoid_gate", dv, dg, tokens * width, plain, None)
    g.sync()
    g.assert_bits_equal(got, plain.get(), "fused gate == stand-alone gate")
    want_c, want_s, want_g = orc.nvfp4_quantize(got, rps)
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32)), "global scales"
    g.assert_bits_equal(scales.get(), want_s, "block scales")
    g.assert_bits_equal(codes.get(), want_c, "codes")
    for d in (out, codes, scales, gs, scratch):
        assert d.guards_intact()


def test_one_scratch_serves_calls_of_any_shape_and_the_error_word_is_sticky(g):
    """The scratch contract: zeroed once by the caller, left zero by every call, so differently shaped
    calls share one buffer back to back with nothing cleared in between; the last word is only ever
    set by the library, never cleared, so a flag planted by the caller survives every call."""
    rng = np.random.default_rng(808)
    H, I = 5120, 17408
    big = 3000
    scratch = g.scratch_for(big, 1)  # the largest any of the calls below needs
    flag = 0x40
    scratch.t[-1] = flag  # planted: must still be there at the end
    plan = [("res", 700, 512), ("gated", 600, 512), ("swiglu", 520, 512), ("res", 2, 0), ("res", 1300, 0),
            ("sig", 700, 512), ("dyn", 33, 16), ("res", 3000, 0), ("gated", 9, 4), ("res", 513, 512)]
    for kind, tokens, rps in plan:
        groups = 1 if rps == 0 else (tokens + rps - 1) // rps
        gs = g.empty_like_dev((groups,), dtype=np.float32)
        if kind == "res":
            left, right = fx.normal_bf16(rng, (tokens, H)), fx.normal_bf16(rng, (tokens, H))
            w = fx.normal_bf16(rng, (H,), 0.02)
            res, out = g.empty_like_dev((tokens, H)), g.empty_like_dev((tokens, H))
            codes, scales = g.empty_like_dev((tokens, H // 2), dtype=np.uint8), g.empty_like_dev((tokens, H // 16), dtype=np.uint8)
            g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4", g.Dev(left), g.Dev(right), g.Dev(w), tokens, H, EPS, rps,
                         res, out, scratch, gs, codes, scales, None)
        elif kind == "gated":
            x, z = fx.normal_bf16(rng, (tokens, 48, 128)), fx.normal_bf16(rng, (tokens, 48, 128))
            w = orc.bf16_encode((0.75 + rng.random(128) * 0.5).astype(np.float32))
            out = g.empty_like_dev((tokens, 6144))
            codes, scales = g.empty_like_dev((tokens, 3072), dtype=np.uint8), g.empty_like_dev((tokens, 384), dtype=np.uint8)
            g.capi.check("q3x_b200_rms_norm_silu_gate_nvfp4", g.Dev(x), g.Dev(w), g.Dev(z), tokens, 48, 128, EPS, rps, out,
                         scratch, gs, codes, scales, None)
        elif kind in ("swiglu", "sig"):
            width = I if kind == "swiglu" else 6144
            a, b = fx.normal_bf16(rng, (tokens, width)), fx.normal_bf16(rng, (tokens, width))
            out = g.empty_like_dev((tokens, width))
            codes = g.empty_like_dev((tokens, width // 2), dtype=np.uint8)
            scales = g.empty_like_dev((tokens, width // 16), dtype=np.uint8)
            g.capi.check("q3x_b200_silu_mul_nvfp4" if kind == "swiglu" else "q3x_b200_sigmoid_gate_nvfp4", g.Dev(a),
                         g.Dev(b), tokens, width, rps, out, scratch, gs, codes, scales, None)
        else:
            x = fx.normal_bf16(rng, (tokens, H))
            out = g.Dev(x)
            codes, scales = g.empty_like_dev((tokens, H // 2), dtype=np.uint8), g.empty_like_dev((tokens, H // 16), dtype=np.uint8)
            g.capi.check("q3x_b200_nvfp4_quantize_dynamic", out, tokens, H, rps, scratch, gs, codes, scales, None)
        g.sync()
        words = scratch.get()
        assert words[-1] == flag, f"{kind} {tokens}/{rps}: the sticky error word was touched ({words[-1]:#x})"
        assert not words[:-1].any(), f"{kind} {tokens}/{rps}: scratch words left non-zero"
        want_c, want_s, want_g = orc.nvfp4_quantize(out.get(), rps)
        g.assert_bits_equal(codes.get(), want_c, f"{kind} {tokens}/{rps}: codes")
        g.assert_bits_equal(scales.get(), want_s, f"{kind} {tokens}/{rps}: scales")
        assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32)), f"{kind} {tokens}/{rps}: global scales"


@pytest.mark.parametrize("rows,cols", [(1, 16), (33, 80), (128, 64), (130, 5120), (512, 6144), (700, 17408)])
def test_swizzled_block_scale_layout_is_a_permutation_of_the_row_major_bytes(g, rows, cols):
    """The 128 x 4 tile layout block-scaled tensor-core MMA reads, against a numpy re-layout of the same
    row-major bytes: every byte lands at tile (r / 128, b / 4), offset (r % 32) * 16 + (r % 128 / 32) * 4 + b % 4;
    the ragged edges are zero."""
    rng = np.random.default_rng([rows, cols, 66])
    blocks = cols // 16
    src = rng.integers(1, 256, size=(rows, blocks), dtype=np.uint8)
    nbytes = g.capi.lib().q3x_b200_nvfp4_swizzled_scale_bytes(rows, cols)
    row_tiles, block_tiles = -(-rows // 128), -(-blocks // 4)
    assert nbytes == row_tiles * block_tiles * 512
    out = g.empty_like_dev((nbytes,), dtype=np.uint8, fill=0xEE)
    g.capi.check("q3x_b200_nvfp4_swizzle_block_scales", g.Dev(src), rows, cols, out, None)
    g.sync()
    want = np.zeros(nbytes, np.uint8)
    r, b = np.meshgrid(np.arange(rows), np.arange(blocks), indexing="ij")
    off = ((r // 128) * block_tiles + b // 4) * 512 + (r % 32) * 16 + (r % 128) // 32 * 4 + b % 4
    want[off.reshape(-1)] = src.reshape(-1)
    g.assert_bits_equal(out.get(), want, "swizzled block scales")
    assert out.guards_intact()
    assert np.array_equal(np.sort(out.get()[out.get() != 0]), np.sort(src.reshape(-1)))  # a permutation plus zero padding
