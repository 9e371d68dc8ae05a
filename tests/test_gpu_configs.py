"""The five benchmark configurations as parity cases, at their stated shapes, through the C ABI.

0. batch-one decode op chain at position 4096 (seed 0);
1. 512-token full-attention chunk: residual+RMSNorm+NVFP4 (tensor amax), q/k head norm + partial RoPE at
   positions 0..511, sigmoid gate, SwiGLU on [512,17408];
2. 8192-token GDN chain: conv1d(k=4)+SiLU over 10240 channels (weights N(0,0.5)), q/k L2 norm, gated
   RMSNorm*silu(z) over 48x128, SwiGLU, NVFP4 of the norm outputs;
3. embedding gather from the 248320x5120 table for 60000 uniform ids, rows partitioned 1/2/4/8 ways;
4. long context: token-sharded runs equal the unsharded run row for row, then a decode step at
   position 131071 with the same weights.
Inputs are seeded synthetic tensors with the stated distributions.
"""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import fixtures as fx

pytestmark = pytest.mark.gpu
EPS = 1e-6
shard = importlib.import_module("qwen3x-orin_b200.shard")


@pytest.fixture(scope="module")
def g():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    return gpu_util


def decode_chain(g, position, seed):
    rng = np.random.default_rng(seed)
    H, I = 5120, 17408
    left, right = fx.normal_bf16(rng, (1, H)), fx.normal_bf16(rng, (1, H))
    w = fx.normal_bf16(rng, (H,), 0.02)
    qg, key = fx.normal_bf16(rng, (1, 24, 2, 256)), fx.normal_bf16(rng, (1, 4, 256))
    qw, kw = fx.normal_bf16(rng, (256,), 0.02), fx.normal_bf16(rng, (256,), 0.02)
    value = fx.normal_bf16(rng, (24 * 256,))
    gate, up = fx.normal_bf16(rng, (I,)), fx.normal_bf16(rng, (I,))
    cos, sin = orc.rope_tables(0, position + 1)

    res, nrm = g.empty_like_dev((1, H)), g.empty_like_dev((1, H))
    g.capi.check("q3x_b200_residual_add_rms_norm", g.Dev(left), g.Dev(right), g.Dev(w), 1, H, EPS, res, nrm, None)
    d_key = g.Dev(key)
    q, gt = g.empty_like_dev((1, 24, 256)), g.empty_like_dev((1, 24, 256))
    g.capi.check("q3x_b200_full_attention_preprocess", g.Dev(qg), d_key, g.Dev(qw), g.Dev(kw), EPS, q, gt, g.Dev(cos),
                 g.Dev(sin), position, 1, None)
    o = g.empty_like_dev((24 * 256,))
    g.capi.check("q3x_b200_sigmoid_gate", g.Dev(value), gt, 24 * 256, o, None)
    h = g.empty_like_dev((I,))
    g.capi.check("q3x_b200_silu_mul", g.Dev(gate), g.Dev(up), I, h, None)
    g.sync()

    want_r, want_n = orc.residual_add_rms_norm(left, right, w, EPS)
    g.assert_bits_equal(res.get(), want_r, "decode residual")
    g.assert_bf16_within(nrm.get(), want_n, 1, 0.98, "decode normalized")
    wq, wg, wk = orc.full_attention_preprocess(qg, key, qw, kw, EPS, cos, sin, position)
    g.assert_bits_equal(gt.get(), wg, "decode gate copy")
    g.assert_bf16_within(q.get()[..., 64:], wq[..., 64:], 1, 0.98, "decode q (pass-through dims)")
    g.assert_bf16_within(d_key.get()[..., 64:], wk[..., 64:], 1, 0.98, "decode k (pass-through dims)")
    # rotated dims: stage-wise on the GPU's own rounded operand (the rotation can amplify a 1-ulp operand change)
    q_n, k_n = g.empty_like_dev((24, 256)), g.Dev(key.reshape(4, 256))
    assert q_n.shape == (24, 256)
    g.capi.check("q3x_b200_rms_norm", g.Dev(np.ascontiguousarray(qg[0, :, 0, :])), g.Dev(qw), 24, 256, EPS, 1, q_n, None)
    g.capi.check("q3x_b200_rms_norm", k_n, g.Dev(kw), 4, 256, EPS, 1, k_n, None)
    g.sync()
    g.assert_bits_equal(q.get()[0], orc.partial_rope(q_n.get(), cos[position], sin[position]), "decode q rotation")
    g.assert_bits_equal(d_key.get()[0], orc.partial_rope(k_n.get(), cos[position], sin[position]), "decode k rotation")
    g.assert_reference_tolerance(q.get(), wq, "decode q end to end", amplified=True)
    g.assert_reference_tolerance(d_key.get(), wk, "decode k end to end", amplified=True)
    g.assert_bf16_within(o.get(), orc.sigmoid_gate(value, wg.reshape(-1)), 1, 0.98, "decode sigmoid gate")
    g.assert_bf16_within(h.get(), orc.silu_mul(gate, up), 1, 0.98, "decode SwiGLU")


def test_config0_decode_chain_at_position_4096(g):
    decode_chain(g, 4096, seed=0)


def test_config1_full_attention_chunk_512(g):
    rng = np.random.default_rng(1)
    T, H, I = 512, 5120, 17408
    left, right = fx.normal_bf16(rng, (T, H)), fx.normal_bf16(rng, (T, H))
    w = fx.normal_bf16(rng, (H,), 0.02)
    res, nrm = g.empty_like_dev((T, H)), g.empty_like_dev((T, H))
    scratch = g.scratch_for(T, 0)
    gs = g.empty_like_dev((1,), dtype=np.float32)
    codes, scales = g.empty_like_dev((T, H // 2), dtype=np.uint8), g.empty_like_dev((T, H // 16), dtype=np.uint8)
    g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4", g.Dev(left), g.Dev(right), g.Dev(w), T, H, EPS, 0, res, nrm,
                 scratch, gs, codes, scales, None)
    qg, key = fx.normal_bf16(rng, (T, 24, 2, 256)), fx.normal_bf16(rng, (T, 4, 256))
    qw, kw = fx.normal_bf16(rng, (256,), 0.02), fx.normal_bf16(rng, (256,), 0.02)
    cos, sin = orc.rope_tables(0, T)
    d_key = g.Dev(key)
    q, gt = g.empty_like_dev((T, 24, 256)), g.empty_like_dev((T, 24, 256))
    g.capi.check("q3x_b200_full_attention_preprocess", g.Dev(qg), d_key, g.Dev(qw), g.Dev(kw), EPS, q, gt, g.Dev(cos),
                 g.Dev(sin), 0, T, None)
    value = fx.normal_bf16(rng, (T, 6144))
    o = g.empty_like_dev((T, 6144))
    g.capi.check("q3x_b200_sigmoid_gate", g.Dev(value), gt, T * 6144, o, None)
    gate, up = fx.normal_bf16(rng, (T, I)), fx.normal_bf16(rng, (T, I))
    h = g.empty_like_dev((T, I))
    g.capi.check("q3x_b200_silu_mul", g.Dev(gate), g.Dev(up), T * I, h, None)
    g.sync()
    want_r, want_n = orc.residual_add_rms_norm(left, right, w, EPS)
    g.assert_bits_equal(res.get(), want_r, "residual")
    g.assert_bf16_within(nrm.get(), want_n, 1, 0.98, "normalized")
    want_c, want_s, want_g = orc.nvfp4_quantize(nrm.get(), 0)   # one global scale from the tensor amax
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32))
    g.assert_bits_equal(codes.get(), want_c, "NVFP4 codes")
    g.assert_bits_equal(scales.get(), want_s, "E4M3 block scales")
    wq, wg, wk = orc.full_attention_preprocess(qg, key, qw, kw, EPS, cos, sin, 0)
    g.assert_bits_equal(gt.get(), wg, "gate copy")
    g.assert_bf16_within(q.get()[..., 64:], wq[..., 64:], 1, 0.98, "q")
    g.assert_bf16_within(d_key.get()[..., 64:], wk[..., 64:], 1, 0.98, "k")
    assert g.ulp_report(q.get()[..., :64], wq[..., :64])[1] > 0.97
    g.assert_reference_tolerance(q.get(), wq, "q end to end", amplified=True)
    g.assert_reference_tolerance(d_key.get(), wk, "k end to end", amplified=True)
    g.assert_bf16_within(o.get(), orc.sigmoid_gate(value, wg.reshape(T, 6144)), 1, 0.98, "sigmoid gate")
    g.assert_bf16_within(h.get(), orc.silu_mul(gate, up), 1, 0.98, "SwiGLU")


def test_config2_gdn_chain_8192(g):
    rng = np.random.default_rng(2)
    T, C_, I = 8192, 10240, 17408
    raw = fx.normal_bf16(rng, (T, C_))
    cw = fx.normal_bf16(rng, (C_, 4), 0.5)
    hist = np.zeros((C_, 3), dtype=np.uint16)
    qs = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    d_raw, d_w = g.Dev(raw), g.Dev(cw)
    conv, fused = g.empty_like_dev((T, C_)), g.empty_like_dev((T, C_))
    h1, h2 = g.Dev(hist), g.Dev(hist)
    g.capi.check("q3x_b200_causal_conv1d_silu", d_raw, T, C_, d_w, h1, conv, None)
    g.capi.check("q3x_b200_causal_conv1d_silu_l2norm", d_raw, T, d_w, h2, EPS, qs, fused, None)
    g.sync()
    want_conv, want_h = orc.causal_conv1d_silu(raw, cw, hist)
    got_conv = conv.get()
    g.assert_bf16_within(got_conv, want_conv, 1, 0.985, "conv")
    g.assert_bits_equal(h1.get(), want_h, "conv history")
    g.assert_bits_equal(h2.get(), want_h, "conv history (fused)")
    got = fused.get()
    g.assert_bits_equal(got[:, 4096:], got_conv[:, 4096:], "v channels")
    g.assert_bf16_within(got[:, :2048].reshape(-1, 128),
                         orc.l2_normalize_heads(got_conv[:, :2048].reshape(-1, 128), EPS, qs), 1, 0.98, "q L2")
    g.assert_bf16_within(got[:, 2048:4096].reshape(-1, 128),
                         orc.l2_normalize_heads(got_conv[:, 2048:4096].reshape(-1, 128), EPS, 1.0), 1, 0.98, "k L2")
    # stand-alone L2 norm entry on the same operand
    l2 = g.empty_like_dev((T * 16, 128))
    g.capi.check("q3x_b200_l2_normalize_heads", g.Dev(np.ascontiguousarray(got_conv[:, 2048:4096]).reshape(-1, 128)),
                 T * 16, 128, EPS, 1.0, l2, None)
    g.sync()
    g.assert_bits_equal(l2.get().reshape(T, 2048), got[:, 2048:4096], "fused k L2 == stand-alone")
    del conv, fused, d_raw

    x, z = fx.normal_bf16(rng, (T, 48, 128)), fx.normal_bf16(rng, (T, 48, 128))
    gw = orc.bf16_encode((0.75 + rng.random(128) * 0.5).astype(np.float32))
    out = g.empty_like_dev((T, 6144))
    scratch = g.scratch_for(T, 512)
    gs = g.empty_like_dev((16,), dtype=np.float32)
    codes, scales = g.empty_like_dev((T, 3072), dtype=np.uint8), g.empty_like_dev((T, 384), dtype=np.uint8)
    g.capi.check("q3x_b200_rms_norm_silu_gate_nvfp4", g.Dev(x), g.Dev(gw), g.Dev(z), T, 48, 128, EPS, 512, out, scratch,
                 gs, codes, scales, None)
    g.sync()
    g.assert_bf16_within(out.get(), orc.rms_norm_rows(x, gw, EPS, centered=False, gate=z).reshape(T, 6144), 1, 0.98,
                         "gated norm")
    want_c, want_s, want_g = orc.nvfp4_quantize(out.get(), 512)
    assert np.array_equal(gs.get().view(np.uint32), want_g.view(np.uint32))
    g.assert_bits_equal(codes.get(), want_c, "NVFP4 codes of the gated norm")
    g.assert_bits_equal(scales.get(), want_s, "block scales of the gated norm")
    del out, codes, scales

    rows = 2048  # SwiGLU is pointwise: a quarter of the panel against the oracle, the rest against itself
    gate, up = fx.normal_bf16(rng, (T, I)), fx.normal_bf16(rng, (T, I))
    h = g.empty_like_dev((T, I))
    d_gate, d_up = g.Dev(gate), g.Dev(up)
    g.capi.check("q3x_b200_silu_mul", d_gate, d_up, T * I, h, None)
    g.sync()
    got_h = h.get()
    g.assert_bf16_within(got_h[:rows], orc.silu_mul(gate[:rows], up[:rows]), 1, 0.98, "SwiGLU")
    h2 = g.empty_like_dev((rows, I))
    g.capi.check("q3x_b200_silu_mul", d_gate.ptr_at(3 * rows * I), d_up.ptr_at(3 * rows * I), rows * I, h2, None)
    g.sync()
    g.assert_bits_equal(h2.get(), got_h[3 * rows:], "SwiGLU is position independent")


def test_config3_embedding_60000_ids_row_partitions(g):
    gen = torch.Generator(device="cuda").manual_seed(3)
    vocab, H, T = 248320, 5120, 60000
    table = (torch.randn((vocab, H), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (T,), generator=gen, device="cuda", dtype=torch.int64)
    ids32 = ids.to(torch.int32)
    out = torch.zeros((T, H), device="cuda", dtype=torch.bfloat16)
    g.capi.check("q3x_b200_embedding_gather", table, vocab, H, ids32, T, out, None)
    g.sync()
    assert torch.equal(out.view(torch.int16), table.index_select(0, ids).view(torch.int16))
    # the whole result against the CPU op
    host_table = table.view(torch.int16).cpu().numpy().view(np.uint16)
    want = orc.embedding_gather(host_table, ids32.cpu().numpy().astype(np.uint32))
    assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)
    del host_table, want
    # row partitions over 1 / 2 / 4 / 8 ranks: each shard's gather is the slice of the whole
    for world in (1, 2, 4, 8):
        parts = shard.partition(T, world)
        assert sum(p.tokens for p in parts) == T
        for p in (parts[0], parts[-1], parts[world // 2]):
            if p.tokens == 0:
                continue
            piece = torch.zeros((p.tokens, H), device="cuda", dtype=torch.bfloat16)
            g.capi.check("q3x_b200_embedding_gather", table, vocab, H, ids32.data_ptr() + 4 * p.first_token, p.tokens,
                         piece, None)
            g.sync()
            assert torch.equal(piece.view(torch.int16), out[p.first_token:p.end_token].view(torch.int16))


def test_config4_sharded_rows_equal_the_unsharded_run_then_decode_at_131071(g):
    gen = torch.Generator(device="cuda").manual_seed(4)
    T, H, C_ = 4096, 5120, 10240   # the sharding rule is size independent; 8 shards of 512 here
    bf = dict(device="cuda", dtype=torch.bfloat16)
    left = torch.randn((T, H), generator=gen, device="cuda").to(torch.bfloat16)
    right = torch.randn((T, H), generator=gen, device="cuda").to(torch.bfloat16)
    w = (torch.randn((H,), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    raw = torch.randn((T, C_), generator=gen, device="cuda").to(torch.bfloat16)
    cw = (torch.randn((C_, 4), generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
    words = g.capi.lib().q3x_b200_nvfp4_scratch_words(T, 512)

    def run(lo, hi, hist):
        n = hi - lo
        res, nrm = torch.empty((n, H), **bf), torch.empty((n, H), **bf)
        scratch = torch.zeros(words, device="cuda", dtype=torch.int32)
        gs = torch.empty(max(1, -(-n // 512)), device="cuda", dtype=torch.float32)
        codes = torch.empty((n, H // 2), device="cuda", dtype=torch.uint8)
        scales = torch.empty((n, H // 16), device="cuda", dtype=torch.uint8)
        g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4", left[lo:hi], right[lo:hi], w, n, H, EPS, 512, res, nrm,
                     scratch, gs, codes, scales, None)
        conv = torch.empty((n, C_), **bf)
        g.capi.check("q3x_b200_causal_conv1d_silu", raw[lo:hi], n, C_, cw, hist, conv, None)
        g.sync()
        return res, nrm, gs, codes, scales, conv

    whole = run(0, T, torch.zeros((C_, 3), **bf))
    for world in (2, 8):
        for p in shard.partition(T, world):
            hist = torch.zeros((C_, 3), **bf)
            halo = p.first_token - p.halo_first
            if halo:
                hist[:, 3 - halo:] = raw[p.halo_first:p.first_token].t()
            part = run(p.first_token, p.end_token, hist.contiguous())
            sl = slice(p.first_token, p.end_token)
            for a, b in zip(part, (whole[0][sl], whole[1][sl], whole[2][p.first_token // 512:-(-p.end_token // 512)],
                                   whole[3][sl], whole[4][sl], whole[5][sl])):
                assert torch.equal(a.view(torch.uint8), b.contiguous().view(torch.uint8))
    # then one batch-one decode step at the last position of the 131072-token prompt
    decode_chain(g, 131071, seed=4)
