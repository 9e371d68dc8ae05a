"""A second opinion on the NVFP4 activation encoder (CPU only).

The reference has no activation quantiser, so the encoder specified in oracle/q3x_oracle.h is this project's own
(parity unpinned).  This test restates the recipe in common use for NVFP4 activations -- the global scale
applied as the multiplier 448 * 6 / amax, a block's E4M3 scale taken from (amax_b / 6) * multiplier, elements
scaled by the reciprocal of (decoded scale / multiplier) -- in numpy FP32, independently of the oracle's C code,
and measures on the benchmark's distributions how often the two formulations pick a different block scale or a
different 4-bit code.  They are the same function in exact arithmetic; in FP32 they differ only where a product
lands next to a rounding boundary, which must be rare, and a differing code must still be a neighbouring one.
The rates are asserted (and documented beside the specification).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import fixtures as fx

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e4m3_rne_sat(x):
    """FP32 -> E4M3 (round to nearest even, saturate at 448) -> code byte, through torch's float8 cast."""
    t = torch.from_numpy(np.clip(x, -448.0, 448.0).astype(np.float32)).to(torch.float8_e4m3fn)
    return t.view(torch.uint8).numpy()


def e2m1_rne_sat(x):
    """FP32 -> E2M1 code (nearest, ties to the even code, saturate at 6); sign in bit 3."""
    mag = np.minimum(np.abs(x), np.float32(6.0))
    # midpoints between neighbouring magnitudes; a tie goes to the code with an even index
    mids = (E2M1[:-1] + E2M1[1:]) / np.float32(2)
    idx = np.searchsorted(mids, mag, side="left").astype(np.int64)          # mag <= mid stays below
    tie = (idx < 7) & (mag == mids[np.minimum(idx, 6)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)                        # tie: move up only onto an even index
    idx = np.where(np.isnan(x), 7, idx)
    return (idx | (np.signbit(x).astype(np.int64) << 3)).astype(np.uint8)


def common_recipe(bits, rows_per_scale):
    """(codes as one nibble per element, block scale bytes, global scales) by the multiplier formulation."""
    x = orc.bf16_decode(bits).astype(np.float32)
    rows, cols = x.shape
    rps = rows if rows_per_scale == 0 else rows_per_scale
    finite = np.where(np.isfinite(x), np.abs(x), np.float32(0))
    nib = np.zeros((rows, cols), np.uint8)
    scales = np.zeros((rows, cols // 16), np.uint8)
    gs = []
    for g0 in range(0, rows, rps):
        sl = slice(g0, min(rows, g0 + rps))
        amax = np.float32(finite[sl].max())
        mult = np.float32(448.0 * 6.0) / amax if amax > 0 else np.float32(1.0)      # encode multiplier
        gs.append(np.float32(1.0) / mult if amax > 0 else np.float32(1.0))
        blk = finite[sl].reshape(-1, cols // 16, 16).max(axis=2)
        sf = e4m3_rne_sat((blk / np.float32(6.0)) * mult)
        scales[sl] = sf
        dec = torch.from_numpy(sf).view(torch.float8_e4m3fn).to(torch.float32).numpy()
        with np.errstate(divide="ignore", invalid="ignore"):
            enc = np.where(dec > 0, np.float32(1.0) / (dec / mult), np.float32(0))
        nib[sl] = e2m1_rne_sat(x[sl] * np.repeat(enc, 16, axis=1))
    return nib, scales, np.array(gs, np.float32)


def oracle_nibbles(bits, rows_per_scale):
    codes, scales, gs = orc.nvfp4_quantize(bits, rows_per_scale)
    nib = np.stack([codes & 0xF, codes >> 4], axis=-1).reshape(bits.shape)
    return nib, scales, gs


@pytest.mark.parametrize("name,shape,std,rps", [("normalised residual rows", (1024, 5120), 1.0, 512),
                                                 ("gated-norm rows", (1024, 6144), 0.6, 512),
                                                 ("SwiGLU rows", (256, 17408), 0.45, 0)])
def test_encoder_agrees_with_the_common_multiplier_recipe(name, shape, std, rps):
    rng = np.random.default_rng([len(name), shape[0], shape[1]])
    bits = fx.normal_bf16(rng, shape, std)
    bits[3, :16] = 0                       # an all-zero block
    ours_n, ours_s, ours_g = oracle_nibbles(bits, rps)
    their_n, their_s, their_g = common_recipe(bits, rps)
    # global scales: amax / 2688 against 1 / (2688 / amax): equal or one FP32 ulp apart
    assert np.all(np.abs(ours_g.view(np.int32) - their_g.view(np.int32)) <= 1)
    scale_diff = float(np.mean(ours_s != their_s))
    code_diff = float(np.mean(ours_n != their_n))
    print(f"{name}: block scales differing {scale_diff:.2e}, codes differing {code_diff:.2e}")
    assert scale_diff < 1e-2 and code_diff < 5e-3, (scale_diff, code_diff)
    # a differing scale is the neighbouring E4M3 code; a differing 4-bit code is a neighbouring magnitude
    ds = np.abs(ours_s.astype(np.int32) - their_s.astype(np.int32))
    assert ds.max() <= 1
    dn = np.abs((ours_n & 7).astype(np.int32) - (their_n & 7).astype(np.int32))
    same_sign = ((ours_n ^ their_n) & 8) == 0
    assert dn.max() <= 1 and np.all(same_sign | ((ours_n & 7) == 0) | ((their_n & 7) == 0))
    # where the block scale agrees the codes agree almost everywhere (x * (1/d) against x * (m / s)); what is
    # left are elements whose scaled value sits on (or within an FP32 rounding of) a midpoint between two E2M1
    # magnitudes -- bf16 inputs are short numbers, so exact ties are not rare -- where the two reciprocals fall
    # on different sides
    same_block = np.repeat(ours_s == their_s, 16, axis=1)
    assert float(np.mean(ours_n[same_block] != their_n[same_block])) < 3e-3


def test_the_two_numpy_encoders_follow_their_definitions():
    """The helpers of this file against the oracle's scalar encoders (which are pinned to the reference's E4M3
    quantiser and value tables), so that a disagreement above is about the recipe, not about a helper."""
    rng = np.random.default_rng(5)
    v = np.concatenate([(rng.standard_normal(20000) * 3).astype(np.float32), E2M1, -E2M1,
                        np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -2.5], np.float32)])
    L = orc.oracle_lib()
    assert np.array_equal(e2m1_rne_sat(v), np.array([L.encode_e2m1(float(x)) for x in v], np.uint8))
    w = np.abs(v) * 40
    assert np.array_equal(e4m3_rne_sat(w), np.array([L.encode_e4m3(float(x)) for x in w], np.uint8))
