"""The MLP block with its projections (chain.ProjectedMlp): residual + RMSNorm + NVFP4 -> gate / up projections
on the block-scaled tensor cores -> SwiGLU + NVFP4 -> down projection, checked stage by stage against the CPU
oracle on the GPU's own previous-stage bytes (the stages' own tests bound each of them; this one checks that the
bytes one stage writes are the bytes the next one reads: codes, swizzled block scales, per-group global scales)."""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
CHUNK = 512


def host(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def dequantised(codes, scales, gs):
    c, s, glob = host(codes), host(scales), host(gs)
    parts = [orc.nvfp4_dequantize(c[i:i + CHUNK], s[i:i + CHUNK], glob[i // CHUNK]) for i in range(0, c.shape[0], CHUNK)]
    return np.concatenate(parts).astype(np.float64)


def assert_projection(got_bits, A, W, what):
    want, mag = A @ W.T, np.abs(A) @ np.abs(W).T
    got = orc.bf16_decode(got_bits).astype(np.float64)
    excess = np.abs(got - want) - (2.0 ** -8 * np.abs(want) + 1e-5 * mag)
    assert np.all(excess <= 0), f"{what}: worst excess {excess.max():.3e}"


def test_projected_mlp_block_stage_by_stage():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    chain = importlib.import_module("qwen3x-orin_b200.chain")
    block = chain.ProjectedMlp(600, torch.device("cuda", 0), hidden=5120, intermediate=1024, seed=5)
    block.enqueue(None)
    torch.cuda.synchronize()
    block.check_error()
    assert not bool(block.scratch.any().item()), "scratch left non-zero"
    # stage 1: residual + norm + NVFP4 against the oracle; codes from the GPU's own normalised rows
    want_r, want_n = orc.residual_add_rms_norm(host(block.left), host(block.right), host(block.norm_w), chain.EPS)
    gpu_util.assert_bits_equal(host(block.residual), want_r, "residual")
    gpu_util.assert_bf16_within(host(block.normalized), want_n, 1, 0.98, "normalized")
    c, s, gs = orc.nvfp4_quantize(host(block.normalized), CHUNK)
    gpu_util.assert_bits_equal(host(block.x_codes), c, "activation codes")
    gpu_util.assert_bits_equal(host(block.x_scales), s, "activation block scales")
    assert np.array_equal(host(block.x_gs).view(np.uint32), gs.view(np.uint32))
    # stage 2: the two projections against the product of the dequantised operands
    X = dequantised(block.x_codes, block.x_scales, block.x_gs)
    weight = lambda w: orc.nvfp4_dequantize(host(w["codes"]), host(w["scales"]), w["scale_2"]).astype(np.float64)
    assert_projection(host(block.gate), X, weight(block.w_gate), "gate projection")
    assert_projection(host(block.up), X, weight(block.w_up), "up projection")
    # stage 3: SwiGLU + NVFP4 on the GPU's own gate / up
    want_h = orc.silu_mul(host(block.gate), host(block.up))
    gpu_util.assert_bf16_within(host(block.h), want_h, 1, 0.98, "SwiGLU")
    c, s, gs = orc.nvfp4_quantize(host(block.h), CHUNK)
    gpu_util.assert_bits_equal(host(block.h_codes), c, "SwiGLU codes")
    gpu_util.assert_bits_equal(host(block.h_scales), s, "SwiGLU block scales")
    assert np.array_equal(host(block.h_gs).view(np.uint32), gs.view(np.uint32))
    # stage 4: the down projection
    Hq = dequantised(block.h_codes, block.h_scales, block.h_gs)
    assert_projection(host(block.down), Hq, weight(block.w_down), "down projection")
    # and the block as a whole stays close to the un-quantised bf16 computation
    f = lambda t: orc.bf16_decode(host(t)).astype(np.float64)
    x = orc.bf16_decode(want_n).astype(np.float64)
    g_, u_ = x @ f(block.w_gate["dense"]).T, x @ f(block.w_up["dense"]).T
    dense = (g_ / (1.0 + np.exp(-g_)) * u_) @ f(block.w_down["dense"]).T
    assert np.corrcoef(f(block.down).reshape(-1), dense.reshape(-1))[0, 1] > 0.97
