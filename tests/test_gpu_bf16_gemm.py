"""GPU test of the bf16 projection of a panel of tokens (q3x_b200_bf16_gemm_bf16), through the C ABI, against the
oracle's batch-one bf16 GEMV (pinned to the reference's bf16_gemv_reference_cpu) per token, with the reference's
acceptance rule for a GEMV row (tests/reference_gemv_cuda_test.cu:36-45) plus the rounding of the bf16 output, and
against the library's own batch-one kernel on the same bytes."""
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


@pytest.mark.parametrize("tokens,n,k", [(1, 8, 8), (7, 48, 5120), (300, 48, 5120), (513, 136, 2064), (64, 6144, 5120)])
def test_bf16_gemm_matches_the_per_token_rule(g, tokens, n, k):
    rng = np.random.default_rng([tokens, n, k, 113])
    x, w = fx.normal_bf16(rng, (tokens, k)), fx.normal_bf16(rng, (n, k), 0.05)
    d_w, d_x = g.Dev(w), g.Dev(x)
    out = g.empty_like_dev((tokens, n))
    g.capi.check("q3x_b200_bf16_gemm_bf16", d_w, d_x, tokens, n, k, out, None, 0, None)
    g.sync()
    wf, xf = orc.bf16_decode(w).astype(np.float64), orc.bf16_decode(x).astype(np.float64)
    want, mag = xf @ wf.T, np.abs(xf) @ np.abs(wf).T
    got = orc.bf16_decode(out.get()).astype(np.float64)
    assert np.all(np.abs(got - want) <= 5.0e-5 * np.sqrt(k) + 5.0e-4 * np.abs(want) + 2.0 ** -8 * np.abs(want))
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-5 * mag + 1e-30)
    one = g.empty_like_dev((n,))
    for t in rng.choice(tokens, size=min(tokens, 4), replace=False):
        want_t = orc.bf16_gemv(w, x[t])
        assert np.all(np.abs(got[t] - want_t) <= 5.0e-5 * np.sqrt(k) + 5.0e-4 * np.abs(want_t) + 2.0 ** -8 * np.abs(want_t))
        g.capi.check("q3x_b200_bf16_gemv", d_w, g.Dev(x[t]), n, k, None, one, None)
        g.sync()
        assert np.mean(out.get()[t] == one.get()) > 0.9
    assert out.guards_intact()


def test_bf16_gemm_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x10000000
    call = lambda **kw: g.capi.call("q3x_b200_bf16_gemm_bf16", kw.get("w", fake), fake + (1 << 24), kw.get("t", 64),
                                    kw.get("n", 64), kw.get("k", 128), kw.get("out", fake + (2 << 24)), None, 0, None)
    assert call(k=12) == inv
    assert call(n=12) == inv
    assert call(w=None) == inv
    assert call(out=fake) == inv
    assert call(t=0) == 0


@pytest.mark.parametrize("tokens,n,k", [(200, 512, 5120), (640, 1024, 5120), (129, 6144, 1024), (96, 48, 5120)])
def test_widened_fp8_weights_through_the_scaled_gemm(g, tokens, n, k):
    """FP8 weights widened to bf16 once (exactly) and multiplied on the dense path with the per-tensor scale in the
    epilogue: the rule of the FP8 projection (tests/test_gpu_fp8_gemm.py) against the float64 product of the decoded
    operands, and the same bytes as the mixed-input FP8 GEMM on nearly every element (both accumulate the same
    products in FP32, in different orders)."""
    rng = np.random.default_rng([tokens, n, k, 127])
    x = fx.normal_bf16(rng, (tokens, k))
    codes = (rng.integers(0x08, 0x78, size=(n, k)) | (rng.integers(0, 2, size=(n, k)) << 7)).astype(np.uint8)
    scale = 0.0123
    d_codes, d_x = g.Dev(codes), g.Dev(x)
    wide = g.empty_like_dev((n, k))
    g.capi.check("q3x_b200_fp8_weights_to_bf16", d_codes, n * k, wide, None)
    g.sync()
    L = orc.oracle_lib()
    want_w = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)[codes]
    assert np.array_equal(orc.bf16_decode(wide.get()), want_w), "E4M3 -> bf16 is exact"
    out, mixed = g.empty_like_dev((tokens, n)), g.empty_like_dev((tokens, n))
    g.capi.check("q3x_b200_bf16_gemm_scaled_bf16", wide, scale, d_x, tokens, n, k, out, None, 0, None)
    g.capi.check("q3x_b200_fp8_gemm_bf16", d_codes, scale, d_x, tokens, n, k, mixed, None, 0, None)
    g.sync()
    xf, wf = orc.bf16_decode(x).astype(np.float64), want_w.astype(np.float64)
    want, mag = (xf @ wf.T) * scale, (np.abs(xf) @ np.abs(wf).T) * scale
    got = orc.bf16_decode(out.get()).astype(np.float64)
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-5 * mag + 1e-30)
    assert np.mean(out.get() == mixed.get()) > 0.97
    assert out.guards_intact() and wide.guards_intact()


def test_widening_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x10000000
    assert g.capi.call("q3x_b200_fp8_weights_to_bf16", fake, 24, fake + (1 << 24), None) == inv      # not 16-element vectors
    assert g.capi.call("q3x_b200_fp8_weights_to_bf16", fake, 64, fake + 32, None) == inv             # overlap
    assert g.capi.call("q3x_b200_fp8_weights_to_bf16", None, 64, fake + (1 << 24), None) == inv
    assert g.capi.call("q3x_b200_fp8_weights_to_bf16", fake, 0, fake + (1 << 24), None) == 0
    assert g.capi.call("q3x_b200_bf16_gemm_scaled_bf16", fake, float("nan"), fake + (1 << 24), 64, 64, 128,
                       fake + (2 << 24), None, 0, None) == inv
