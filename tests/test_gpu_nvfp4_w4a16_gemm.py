"""GPU test of the weight-only NVFP4 projection of a panel of tokens (q3x_b200_nvfp4_w4a16_gemm_bf16), through the
C ABI, against the oracle's batch-one NVFP4 GEMV (pinned to the reference's nvfp4_gemv_reference_cpu) applied
per token, with the reference's acceptance rule for a GEMV row (tests/reference_gemv_cuda_test.cu:36-45) plus the
rounding of the bf16 output, and against the library's own batch-one kernel on the same bytes."""
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


@pytest.mark.parametrize("tokens,n,k", [(1, 8, 32), (7, 48, 512), (64, 1024, 5120), (512, 640, 5120), (256, 5120, 17408),
                                        (513, 144, 2080)])
def test_w4a16_gemm_matches_the_per_token_rule(g, tokens, n, k):
    rng = np.random.default_rng([tokens, n, k, 107])
    x = fx.normal_bf16(rng, (tokens, k))
    packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = rng.integers(0x08, 0x68, size=(n, k // 16), dtype=np.uint8)  # subnormal and normal E4M3 scales
    scale_2 = 0.004
    d_p, d_s, d_x = g.Dev(packed), g.Dev(scales), g.Dev(x)
    d_st = g.empty_like_dev((k // 16, n))
    g.capi.check("q3x_b200_nvfp4_transpose_block_scales", d_s, n, k, d_st, None)
    g.sync()
    L = orc.oracle_lib()
    e4 = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    g.assert_bits_equal(d_st.get(), orc.bf16_encode(e4[scales.T]), "transposed block scales as bf16")
    need = g.capi.lib().q3x_b200_nvfp4_w4a16_gemm_workspace_bytes(tokens, n, k)
    ws, out = g.empty_like_dev((max(need, 256),), dtype=np.uint8), g.empty_like_dev((tokens, n))
    g.capi.check("q3x_b200_nvfp4_w4a16_gemm_bf16", d_p, d_st, scale_2, d_x, tokens, n, k, out, ws, need, None)
    g.sync()
    deq = orc.nvfp4_dequantize(packed, scales, scale_2).astype(np.float64)
    xf = orc.bf16_decode(x).astype(np.float64)
    want, mag = xf @ deq.T, np.abs(xf) @ np.abs(deq).T
    got = orc.bf16_decode(out.get()).astype(np.float64)
    assert np.all(np.abs(got - want) <= 5.0e-5 * np.sqrt(k) + 5.0e-4 * np.abs(want) + 2.0 ** -8 * np.abs(want))
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-5 * mag + 1e-30)
    rows = rng.choice(tokens, size=min(tokens, 4), replace=False)
    one = g.empty_like_dev((n,))
    for t in rows:
        want_t = orc.nvfp4_gemv(packed, scales, scale_2, x[t])
        assert np.all(np.abs(got[t] - want_t) <= 5.0e-5 * np.sqrt(k) + 5.0e-4 * np.abs(want_t) + 2.0 ** -8 * np.abs(want_t))
        g.capi.check("q3x_b200_nvfp4_gemv", d_p, d_s, scale_2, g.Dev(x[t]), n, k, None, one, None)
        g.sync()
        assert np.mean(out.get()[t] == one.get()) > 0.9
    assert out.guards_intact() and ws.guards_intact()


def test_w4a16_gemm_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x10000000
    call = lambda **kw: g.capi.call("q3x_b200_nvfp4_w4a16_gemm_bf16", kw.get("w", fake), fake + (1 << 24), kw.get("s", 0.5),
                                    fake + (2 << 24), kw.get("t", 64), kw.get("n", 64), kw.get("k", 256),
                                    kw.get("out", fake + (3 << 24)), None, 0, None)
    assert call(k=48) == inv
    assert call(n=12) == inv
    assert call(s=-0.5) == inv
    assert call(w=None) == inv
    assert call(out=fake) == inv
    assert call(t=0) == 0


@pytest.mark.parametrize("tokens,n,k", [(200, 512, 5120), (130, 5120, 1024), (64, 48, 512)])
def test_widened_nvfp4_weights_through_the_scaled_dense_gemm(g, tokens, n, k):
    """An NVFP4 weight widened to bf16 once (code x block scale, exact) and multiplied on the dense path with the
    second-level scale in the epilogue: the widened bytes equal the oracle's dequantisation at scale 1, the product
    obeys the rule above, and nearly every output byte equals the weight-only kernel's (same products, FP32 sums in
    another order)."""
    rng = np.random.default_rng([tokens, n, k, 131])
    x = fx.normal_bf16(rng, (tokens, k))
    packed = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = rng.integers(0x08, 0x68, size=(n, k // 16), dtype=np.uint8)
    scales[0, 0] |= 0x80  # a negative block scale
    scale_2 = 0.004
    d_p, d_s, d_x = g.Dev(packed), g.Dev(scales), g.Dev(x)
    wide = g.empty_like_dev((n, k))
    g.capi.check("q3x_b200_nvfp4_weights_to_bf16", d_p, d_s, n, k, wide, None)
    g.sync()
    unit = orc.nvfp4_dequantize(packed, scales, 1.0).astype(np.float32)
    assert np.array_equal(orc.bf16_decode(wide.get()), unit), "code x block scale is exact in bf16"
    out = g.empty_like_dev((tokens, n))
    g.capi.check("q3x_b200_bf16_gemm_scaled_bf16", wide, scale_2, d_x, tokens, n, k, out, None, 0, None)
    d_st = g.empty_like_dev((k // 16, n))
    g.capi.check("q3x_b200_nvfp4_transpose_block_scales", d_s, n, k, d_st, None)
    need = g.capi.lib().q3x_b200_nvfp4_w4a16_gemm_workspace_bytes(tokens, n, k)
    ws, mixed = g.empty_like_dev((max(need, 256),), dtype=np.uint8), g.empty_like_dev((tokens, n))
    g.capi.check("q3x_b200_nvfp4_w4a16_gemm_bf16", d_p, d_st, scale_2, d_x, tokens, n, k, mixed, ws, need, None)
    g.sync()
    deq, xf = unit.astype(np.float64) * scale_2, orc.bf16_decode(x).astype(np.float64)
    want, mag = xf @ deq.T, np.abs(xf) @ np.abs(deq).T
    got = orc.bf16_decode(out.get()).astype(np.float64)
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-5 * mag + 1e-30)
    assert np.mean(out.get() == mixed.get()) > 0.97
    assert out.guards_intact() and wide.guards_intact()
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x10000000
    assert g.capi.call("q3x_b200_nvfp4_weights_to_bf16", fake, fake + (1 << 24), 8, 24, fake + (2 << 24), None) == inv
    assert g.capi.call("q3x_b200_nvfp4_weights_to_bf16", fake, fake + (1 << 24), 8, 32, fake + 64, None) == inv
    assert g.capi.call("q3x_b200_nvfp4_weights_to_bf16", fake, None, 8, 32, fake + (2 << 24), None) == inv
    assert g.capi.call("q3x_b200_nvfp4_weights_to_bf16", fake, fake + (1 << 24), 0, 32, fake + (2 << 24), None) == 0
