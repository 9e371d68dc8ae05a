"""One full-attention layer with its projections (chain.ProjectedAttentionLayer), checked stage by stage against the
CPU oracle on the GPU's own previous-stage bytes: residual + RMSNorm, the FP8 q|gate / k / v projections (k and v
written into the KV caches), q / k head norm + RoPE (keys in place in the cache), bulk causal attention + sigmoid
gate over the cache, the FP8 output projection, and the hand-over to the MLP block.  The stages' own tests bound
each kernel; this one checks that the bytes one stage writes are the bytes the next one reads."""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def host(t):
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def assert_fp8_projection(got_bits, x_bits, weight, what):
    L = orc.oracle_lib()
    e4 = np.array([L.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    wf = (e4[host(weight["codes"])] * np.float32(weight["scale"])).astype(np.float64)
    xf = orc.bf16_decode(x_bits).astype(np.float64)
    want, mag = xf @ wf.T, np.abs(xf) @ np.abs(wf).T
    got = orc.bf16_decode(got_bits).astype(np.float64)
    excess = np.abs(got - want) - (2.0 ** -8 * np.abs(want) + 2e-5 * mag + 1e-30)
    assert np.all(excess <= 0), f"{what}: worst excess {excess.max():.3e}"


def test_full_attention_layer_stage_by_stage():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    capi = gpu_util.capi
    chain = importlib.import_module("qwen3x-orin_b200.chain")
    tokens, first = 200, 120
    layer = chain.ProjectedAttentionLayer(tokens, first, torch.device("cuda", 0), intermediate=1024, seed=9)
    old_keys, old_values = host(layer.key_cache[:first]), host(layer.value_cache[:first])
    layer.enqueue(None)
    torch.cuda.synchronize()
    layer.mlp.check_error()
    # stage 1: residual + norm
    want_r, want_n = orc.residual_add_rms_norm(host(layer.residual_in), host(layer.previous_mlp_out), host(layer.input_norm_w),
                                               chain.EPS)
    gpu_util.assert_bits_equal(host(layer.residual_mid), want_r, "residual")
    gpu_util.assert_bf16_within(host(layer.normalized), want_n, 1, 0.98, "normalized")
    x = host(layer.normalized)
    # stage 2: projections; the caches keep what was there before the tile
    assert_fp8_projection(host(layer.q_gate), x, layer.w_q, "q|gate projection")
    assert_fp8_projection(host(layer.value_cache[first:]).reshape(tokens, -1), x, layer.w_v, "v projection into the cache")
    gpu_util.assert_bits_equal(host(layer.key_cache[:first]), old_keys, "earlier keys untouched")
    gpu_util.assert_bits_equal(host(layer.value_cache[:first]), old_values, "earlier values untouched")
    raw_key = torch.empty((tokens, 1024), device="cuda", dtype=torch.bfloat16)  # the k projection again: same bytes
    capi.check("q3x_b200_fp8_gemm_bf16", layer.w_k["codes"], layer.w_k["scale"], layer.normalized, tokens, 1024, 5120, raw_key,
               None, 0, None)
    torch.cuda.synchronize()
    assert_fp8_projection(host(raw_key), x, layer.w_k, "k projection")
    # stage 3: head norms + RoPE on the GPU's projections (two roundings in the rotated dims: the quota form)
    q_want, g_want, k_want = orc.full_attention_preprocess(host(layer.q_gate).reshape(tokens, 24, 2, 256), host(raw_key).reshape(tokens, 4, 256),
                                                           host(layer.q_norm_w), host(layer.k_norm_w), chain.EPS,
                                                           layer.cos.cpu().numpy(), layer.sin.cpu().numpy(), first)
    gpu_util.assert_bits_equal(host(layer.gate_out), g_want, "gate")
    gpu_util.assert_reference_tolerance(host(layer.q_out), q_want, "q after norm + RoPE", amplified=True)
    gpu_util.assert_reference_tolerance(host(layer.key_cache[first:]), k_want, "k after norm + RoPE, in the cache", amplified=True)
    assert gpu_util.ulp_report(host(layer.q_out), q_want)[1] > 0.97
    # stage 4: attention over the cache as it now stands, token by token
    kc, vc, q, gate = host(layer.key_cache), host(layer.value_cache), host(layer.q_out), host(layer.gate_out)
    want_a = np.stack([orc.gqa_attention(q[t], kc[:first + t + 1], vc[:first + t + 1], 0.0625, gate=gate[t])[0]
                       for t in range(tokens)])
    gpu_util.assert_sum_within(host(layer.attention), want_a, 3, 1e-5, 0.98, "attention")
    gpu_util.assert_reference_tolerance(host(layer.attention), want_a, "attention", amplified=True)
    # stage 5: output projection, and the MLP block's first operator took it as its right operand
    assert_fp8_projection(host(layer.attention_projected), host(layer.attention).reshape(tokens, -1), layer.w_o, "output projection")
    want_r2, _ = orc.residual_add_rms_norm(host(layer.residual_mid), host(layer.attention_projected), host(layer.mlp.norm_w),
                                           chain.EPS)
    gpu_util.assert_bits_equal(host(layer.mlp.residual), want_r2, "post-attention residual")
    assert bool(torch.isfinite(layer.mlp.down.float()).all().item())
