"""GPU test of the weight-only FP8 projection of a panel of tokens (q3x_b200_fp8_gemm_bf16), through the C ABI,
against the reference's batch-one rule applied per token: sum over columns of (decode(w) * scale) * x in float64,
with the reference's acceptance rule for a GEMV row (tests/reference_gemv_cuda_test.cu:36-45) plus the rounding of
the bf16 output, and against the library's own batch-one kernel on the same bytes."""
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


@pytest.mark.parametrize("tokens,n,k", [(1, 8, 16), (7, 24, 160), (64, 1024, 5120), (512, 640, 5120), (300, 5120, 6144),
                                        (513, 136, 2064)])
def test_fp8_gemm_matches_the_per_token_rule(g, tokens, n, k):
    rng = np.random.default_rng([tokens, n, k, 103])
    x = fx.normal_bf16(rng, (tokens, k))
    w8 = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    w8[(w8 & 0x7F) == 0x7F] = 0x3C  # no NaN codes
    scale = 0.0123
    need = g.capi.lib().q3x_b200_fp8_gemm_workspace_bytes(tokens, n, k)
    d_w, d_x = g.Dev(w8), g.Dev(x)
    ws, out = g.empty_like_dev((max(need, 256),), dtype=np.uint8), g.empty_like_dev((tokens, n))
    g.capi.check("q3x_b200_fp8_gemm_bf16", d_w, scale, d_x, tokens, n, k, out, ws, need, None)
    g.sync()
    L = orc.oracle_lib()
    e4 = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    wf = (e4[w8] * np.float32(scale)).astype(np.float64)
    xf = orc.bf16_decode(x).astype(np.float64)
    want, mag = xf @ wf.T, np.abs(xf) @ np.abs(wf).T
    got = orc.bf16_decode(out.get()).astype(np.float64)
    assert np.all(np.abs(got - want) <= 5.0e-5 * np.sqrt(k) + 5.0e-4 * np.abs(want) + 2.0 ** -8 * np.abs(want))
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 2e-5 * mag + 1e-30)
    # the batch-one kernel on the same bytes, token by token: the same value up to the accumulation order
    rows = rng.choice(tokens, size=min(tokens, 5), replace=False)
    one = g.empty_like_dev((n,))
    for t in rows:
        g.capi.check("q3x_b200_fp8_gemv", d_w, scale, g.Dev(x[t]), n, k, None, one, None)
        g.sync()
        single = orc.bf16_decode(one.get()).astype(np.float64)
        assert np.all(np.abs(got[t] - single) <= 2.0 ** -7 * np.abs(single) + 4e-5 * mag[t] + 1e-30)
        assert np.mean(out.get()[t] == one.get()) > 0.9
    assert out.guards_intact() and ws.guards_intact()


def test_fp8_gemm_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x10000000
    call = lambda **kw: g.capi.call("q3x_b200_fp8_gemm_bf16", kw.get("w", fake), kw.get("s", 0.5), fake + (1 << 24),
                                    kw.get("t", 64), kw.get("n", 64), kw.get("k", 128), kw.get("out", fake + (2 << 24)),
                                    fake + (3 << 24), kw.get("wsb", 1 << 20), None)
    assert call(k=120) == inv
    assert call(n=12) == inv
    assert call(s=float("nan")) == inv
    assert call(w=None) == inv
    assert call(out=fake) == inv
    assert call(t=0) == 0
    assert g.capi.lib().q3x_b200_fp8_gemm_workspace_bytes(0, 64, 128) == 0
