"""GPU test of the projection that consumes the NVFP4 activations (q3x_b200_nvfp4_gemm_bf16), through the C ABI.

The operands are produced by the library's own quantiser (codes, row-major block scales, global scales per
scale group), the block scales are re-laid out by q3x_b200_nvfp4_swizzle_block_scales, and the result is
compared with the product of the two DEQUANTISED operands computed on the CPU in float64 (oracle's decoder, which
is pinned to the reference's).  Every product of two codes and two block scales is exact in FP32, so what
separates the kernel from that product is the FP32 accumulation order and one rounding to bf16:
|got - want| <= 2^-8 |want| + 1e-5 sum |a||w|.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import fixtures as fx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    return gpu_util


def quantised(g, values, rows_per_scale):
    """bf16 matrix -> (codes, row-major scales, swizzled scales, global scales) on the device."""
    rows, cols = values.shape
    groups = 1 if rows_per_scale == 0 else (rows + rows_per_scale - 1) // rows_per_scale
    codes = g.empty_like_dev((rows, cols // 2), dtype=np.uint8)
    scales = g.empty_like_dev((rows, cols // 16), dtype=np.uint8)
    gs = g.empty_like_dev((groups,), dtype=np.float32)
    g.capi.check("q3x_b200_nvfp4_quantize_dynamic", g.Dev(values), rows, cols, rows_per_scale,
                 g.scratch_for(rows, rows_per_scale), gs, codes, scales, None)
    nbytes = g.capi.lib().q3x_b200_nvfp4_swizzled_scale_bytes(rows, cols)
    swizzled = g.empty_like_dev((nbytes,), dtype=np.uint8)
    g.capi.check("q3x_b200_nvfp4_swizzle_block_scales", scales, rows, cols, swizzled, None)
    g.sync()
    return codes, scales, swizzled, gs


def dequantised(codes, scales, gs, rows_per_scale):
    c, s, glob = codes.get(), scales.get(), gs.get()
    rows = c.shape[0]
    step = rows if rows_per_scale == 0 else rows_per_scale
    parts = [orc.nvfp4_dequantize(c[i:i + step], s[i:i + step], glob[i // step]) for i in range(0, rows, step)]
    return np.concatenate(parts).astype(np.float64)


@pytest.mark.parametrize("tokens,n,k,rps", [(128, 128, 64, 0), (37, 8, 128, 0), (512, 256, 1024, 512),
                                            (1300, 384, 5120, 512), (640, 1032, 6144, 128), (300, 17408, 320, 0), (777, 136, 2048, 100)])
def test_nvfp4_gemm_matches_the_dequantised_product(g, tokens, n, k, rps):
    rng = np.random.default_rng([tokens, n, k, 101])
    a = fx.normal_bf16(rng, (tokens, k)) if rps == 0 else orc.bf16_encode(
        (rng.standard_normal((tokens, k)) * np.exp2(rng.integers(-3, 4, size=(tokens, 1)))).astype(np.float32))
    w = fx.normal_bf16(rng, (n, k), 0.04)
    a_codes, a_scales, a_swz, a_gs = quantised(g, a, rps)
    w_codes, w_scales, w_swz, w_gs = quantised(g, w, 0)
    w_scale_2 = float(w_gs.get()[0])
    need = g.capi.lib().q3x_b200_nvfp4_gemm_workspace_bytes(tokens, n, k, rps)
    assert need > 0
    ws = g.empty_like_dev((need,), dtype=np.uint8)
    out = g.empty_like_dev((tokens, n))
    g.capi.check("q3x_b200_nvfp4_gemm_bf16", a_codes, a_swz, a_gs, rps, w_codes, w_swz, w_scale_2, tokens, n, k, out, ws,
                 need, None)
    g.sync()
    A, W = dequantised(a_codes, a_scales, a_gs, rps), dequantised(w_codes, w_scales, w_gs, 0)
    want = A @ W.T
    mag = np.abs(A) @ np.abs(W).T
    got = orc.bf16_decode(out.get()).astype(np.float64)
    excess = np.abs(got - want) - (2.0 ** -8 * np.abs(want) + 1e-5 * mag)
    assert np.all(excess <= 0), f"worst excess {excess.max():.3e} at {np.unravel_index(excess.argmax(), excess.shape)}"
    # 4-bit operands: close to the bf16 product, not equal
    exact = orc.bf16_decode(a).astype(np.float64) @ orc.bf16_decode(w).astype(np.float64).T
    assert np.corrcoef(got.reshape(-1), exact.reshape(-1))[0, 1] > 0.98
    for d in (out, ws, a_codes, a_swz, w_codes, w_swz):
        assert d.guards_intact()


def test_nvfp4_gemm_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x10000000
    args = lambda **kw: [kw.get("a", fake), fake + (1 << 24), fake + (2 << 24), kw.get("rps", 0), fake + (3 << 24),
                         fake + (4 << 24), kw.get("s2", 0.5), kw.get("t", 256), kw.get("n", 64), kw.get("k", 128),
                         kw.get("out", fake + (5 << 24)), kw.get("ws", fake + (6 << 24)), kw.get("wsb", 1 << 20), None]
    call = lambda **kw: g.capi.call("q3x_b200_nvfp4_gemm_bf16", *args(**kw))
    assert call(k=96) == inv            # in_features not a multiple of 64
    assert call(n=12) == inv            # out_features not a multiple of 8
    assert call(s2=-1.0) == inv
    assert call(a=None) == inv
    assert call(wsb=8) == inv           # workspace too small
    assert call(out=fake) == inv        # output on the activation codes
    assert call(t=0) == 0
    assert g.capi.lib().q3x_b200_nvfp4_gemm_workspace_bytes(0, 64, 128, 0) == 0
