"""One gated-delta-net layer with its projections (chain.ProjectedGdnLayer), checked stage by stage against the CPU
oracle on the GPU's own previous-stage bytes: residual + RMSNorm, the FP8 qkv / z projections, causal conv1d + SiLU
with its history, the token-sequential recurrence with its state, the gated RMSNorm + NVFP4, the NVFP4 output
projection, and the hand-over to the MLP block."""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.test_gpu_attention_layer import assert_fp8_projection, host

pytestmark = pytest.mark.gpu
CHUNK = 512


def test_gdn_layer_stage_by_stage():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    chain = importlib.import_module("qwen3x-orin_b200.chain")
    tokens = 150
    layer = chain.ProjectedGdnLayer(tokens, torch.device("cuda", 0), intermediate=1024, seed=13)
    state0, history0 = host(layer.state).copy(), host(layer.conv_history).copy()
    layer.enqueue(None)
    torch.cuda.synchronize()
    layer.check_error()
    want_r, want_n = orc.residual_add_rms_norm(host(layer.residual_in), host(layer.previous_mlp_out), host(layer.input_norm_w),
                                               chain.EPS)
    gpu_util.assert_bits_equal(host(layer.residual_mid), want_r, "residual")
    gpu_util.assert_bf16_within(host(layer.normalized), want_n, 1, 0.98, "normalized")
    x = host(layer.normalized)
    assert_fp8_projection(host(layer.qkv), x, layer.w_qkv, "qkv projection")
    assert_fp8_projection(host(layer.z), x, layer.w_z, "z projection")
    for name, got_t, w_t in (("a", layer.a, layer.w_a), ("b", layer.b, layer.w_b)):
        wf, xf = orc.bf16_decode(host(w_t)).astype(np.float64), orc.bf16_decode(x).astype(np.float64)
        want, mag = xf @ wf.T, np.abs(xf) @ np.abs(wf).T
        got = orc.bf16_decode(host(got_t)).astype(np.float64)
        assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-5 * mag + 1e-30), f"{name} gate projection"
    # conv on the GPU's own projection, history carried out
    conv_want, hist_want = orc.causal_conv1d_silu(host(layer.qkv), host(layer.conv_w), history0)
    gpu_util.assert_bf16_within(host(layer.conv_out), conv_want, 1, 0.98, "conv")
    gpu_util.assert_bits_equal(host(layer.conv_history), hist_want, "conv history")
    # recurrence on the GPU's own conv output: the rule of the recurrence's own test (multi-token: the bf16 state feeds
    # back, so the reference's acceptance rule is the bound and most elements are exact)
    core_want, state_want = orc.gated_delta_net_update(host(layer.conv_out), host(layer.a), host(layer.b), host(layer.A_log),
                                                       host(layer.dt_bias), state0, chain.EPS)
    gpu_util.assert_reference_tolerance(host(layer.core), core_want, "recurrence output", amplified=True)
    # the state feeds back into itself across a bf16 boundary 150 times: nearly all elements exact, the rest within a
    # rounding-level fraction of the state's largest magnitude (the recurrence's own test uses the same rule)
    got_state = host(layer.state)
    assert gpu_util.ulp_report(got_state, state_want)[1] > 0.99
    a_, e_ = orc.bf16_decode(got_state).astype(np.float64), orc.bf16_decode(state_want).astype(np.float64)
    assert np.max(np.abs(a_ - e_)) <= 2.0 ** -7 * np.max(np.abs(e_))
    assert gpu_util.ulp_report(host(layer.core), core_want)[1] > 0.9
    # gated norm + NVFP4 on the GPU's own recurrence output and z
    gated_want = orc.rms_norm_rows(host(layer.core).reshape(tokens, 48, 128), host(layer.gdn_norm_w), chain.EPS, centered=False,
                                   gate=host(layer.z).reshape(tokens, 48, 128)).reshape(tokens, -1)
    gpu_util.assert_bf16_within(host(layer.gated), gated_want, 1, 0.98, "gated norm")
    c, s, gs = orc.nvfp4_quantize(host(layer.gated), CHUNK)
    gpu_util.assert_bits_equal(host(layer.gated_codes), c, "codes")
    gpu_util.assert_bits_equal(host(layer.gated_scales), s, "block scales")
    # output projection against the product of the dequantised operands
    A = orc.nvfp4_dequantize(c, s, gs[0]).astype(np.float64)
    W = orc.nvfp4_dequantize(host(layer.w_o["codes"]), host(layer.w_o["scales"]), layer.w_o["scale_2"]).astype(np.float64)
    want, mag = A @ W.T, np.abs(A) @ np.abs(W).T
    got = orc.bf16_decode(host(layer.mixer_projected)).astype(np.float64)
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-5 * mag)
    want_r2, _ = orc.residual_add_rms_norm(host(layer.residual_mid), host(layer.mixer_projected), host(layer.mlp.norm_w), chain.EPS)
    gpu_util.assert_bits_equal(host(layer.mlp.residual), want_r2, "post-mixer residual")
    assert bool(torch.isfinite(layer.mlp.down.float()).all().item())


def test_gdn_layer_with_the_chunked_recurrence():
    """The same layer with the recurrence in 64-token chunks: its output and state against the sequential oracle on
    the GPU's own conv output, by the figures the reference uses for this form (NRMSE, cosine; the oracle's per-token
    state rounding alone puts it about 7e-3 from the unrounded recurrence over 150 tokens), and the stage after it
    exact on the GPU's own bytes."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util
    from tests.test_gpu_gdn_chunked import figures

    orc.build()
    gpu_util.capi.load()
    chain = importlib.import_module("qwen3x-orin_b200.chain")
    tokens = 150
    layer = chain.ProjectedGdnLayer(tokens, torch.device("cuda", 0), intermediate=1024, seed=13, chunked=True)
    state0 = host(layer.state).copy()
    layer.enqueue(None)
    torch.cuda.synchronize()
    layer.check_error()
    core_want, state_want = orc.gated_delta_net_update(host(layer.conv_out), host(layer.a), host(layer.b), host(layer.A_log),
                                                       host(layer.dt_bias), state0, chain.EPS)
    dec = lambda x: orc.bf16_decode(x).astype(np.float64)
    nrmse, cosine, _ = figures(dec(host(layer.core)), dec(core_want))
    assert nrmse <= 1.2e-2 and cosine >= 0.9995, (nrmse, cosine)
    nrmse, cosine, _ = figures(dec(host(layer.state)), dec(state_want))
    assert nrmse <= 1.2e-2 and cosine >= 0.9995, (nrmse, cosine)
    gated_want = orc.rms_norm_rows(host(layer.core).reshape(tokens, 48, 128), host(layer.gdn_norm_w), chain.EPS, centered=False,
                                   gate=host(layer.z).reshape(tokens, 48, 128)).reshape(tokens, -1)
    gpu_util.assert_bf16_within(host(layer.gated), gated_want, 1, 0.98, "gated norm")
    c, s, _ = orc.nvfp4_quantize(host(layer.gated), CHUNK)
    gpu_util.assert_bits_equal(host(layer.gated_codes), c, "codes")
    gpu_util.assert_bits_equal(host(layer.gated_scales), s, "block scales")
    assert bool(torch.isfinite(layer.mlp.down.float()).all().item())
