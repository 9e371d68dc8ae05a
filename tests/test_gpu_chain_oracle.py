"""The benchmark's operator chain (`LayerStack.enqueue_step`) against the CPU oracle, as a CHAIN.

Configuration 3 (embedding gather of 60000 uniformly drawn ids from the 248320 x 5120 table, then the
per-layer op chains, rows partitioned 1/2/4/8 ways) and configuration 4 (the long prompt) run the very
same chain; here it runs over the first four layers (GDN, GDN, GDN, full attention -- one full period of
the layer pattern) at 60000 tokens, and every tensor the chain leaves behind is checked on sampled rows
against the oracle's call sequence for that row:

    embedding -> per layer [ residual add + centred RMSNorm (+NVFP4) -> conv1d+SiLU -> q/k L2 norm ->
    gated RMSNorm*silu(z) (+NVFP4)   |   split + q/k head norm + partial RoPE -> sigmoid gate ]
    -> residual add + centred RMSNorm (+NVFP4) -> SwiGLU

The rows are sampled from each of the eight shards of the 8-way row partition (first and last row of
every shard, rows next to 512-token chunk borders, random rows), so the check covers what every rank of
the sharded run computes.  Tolerances: residual stream, embedding rows and gate copy bit-exact; every
other bf16 output within 1 bf16 ulp (the rotated dims and the conv -> L2 chain, two roundings in a row,
within the reference's own tolerance as a hard bound); NVFP4 codes, block scales and global scales
bit-exact given the GPU's own normalised rows.
"""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
chain = importlib.import_module("qwen3x-orin_b200.chain")
shard = importlib.import_module("qwen3x-orin_b200.shard")


@pytest.fixture(scope="module")
def g():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    return gpu_util


def bits(t):
    if t.dtype == torch.uint8:
        return t.contiguous().cpu().numpy()
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def sample_rows(total, world, rng, per_shard=64):
    rows = set()
    for p in shard.partition(total, world):
        if p.tokens == 0:
            continue
        border = [p.first_token, p.first_token + 1, p.first_token + 2, p.end_token - 1]
        chunk_edges = [c for c in range(p.first_token, p.end_token, 512)][1:3]
        near = [e + d for e in chunk_edges for d in (-1, 0, 1, 2)]
        rnd = rng.integers(p.first_token, p.end_token, size=per_shard - len(border) - len(near))
        rows.update(int(r) for r in border + near + list(rnd) if p.first_token <= r < p.end_token)
    return np.array(sorted(rows), dtype=np.int64)


def test_configs_3_and_4_first_layer_period_against_the_oracle_chain(g):
    total, layers = 60000, 4
    stack = chain.LayerStack(total, first_position=0, seed=33, layers=layers)  # the full 248320-row table
    stream = torch.cuda.current_stream().cuda_stream
    final = stack.residual[stack.enqueue_step(stream)]
    torch.cuda.synchronize()
    stack.check_error("chain under test")

    rng = np.random.default_rng(3344)
    rows = sample_rows(total, 8, rng)
    assert rows.size >= 8 * 48
    idx = torch.from_numpy(rows).cuda()

    def take(t):
        return bits(t.index_select(0, idx))

    inp = {n: take(t) for n, t in stack.inputs.items() if n not in ("conv_raw", "key")}
    # (the key rows are updated in place by the full-attention layer; they have a test of their own below)
    ids = stack.token_ids.index_select(0, idx).cpu().numpy().astype(np.uint32)
    table_rows = bits(stack.table.index_select(0, torch.from_numpy(ids.astype(np.int64)).cuda()))
    norm_w, q_w, k_w = bits(stack.norm_w), bits(stack.q_norm_w), bits(stack.k_norm_w)
    gdn_w, conv_w = bits(stack.gdn_norm_w), bits(stack.conv_w)
    # the cos / sin tables are INPUTS of the operator: the oracle gets the very tables the chain used (they
    # follow the reference's recipe; torch's and libm's cosf differ in the last FP32 bit now and then, which
    # the bf16 round trip of the recipe mostly, not always, hides)
    cos, sin = stack.cos.cpu().numpy(), stack.sin.cpu().numpy()
    ref_cos, ref_sin = orc.rope_tables(0, total)
    assert np.mean(cos == ref_cos) > 0.999 and np.mean(sin == ref_sin) > 0.999, "tables drifted from the recipe"

    # three raw rows of history for every sampled row (zeros before the prompt starts)
    raw = stack.inputs["conv_raw"]
    hist_idx = (idx[:, None] + torch.arange(-3, 1, device="cuda")[None, :])
    window = bits(raw.index_select(0, hist_idx.clamp(min=0).reshape(-1))).reshape(rows.size, 4, -1)
    window[hist_idx.cpu().numpy() < 0] = 0

    EPS = chain.EPS
    qs = float(np.float32(1.0) / np.sqrt(np.float32(128.0)))
    residual = orc.embedding_gather(table_rows, np.arange(rows.size, dtype=np.uint32))
    assert np.array_equal(residual, table_rows)
    want = {}
    for layer in range(layers):
        residual, want["normalized"] = orc.residual_add_rms_norm(residual, inp["proj_out"], norm_w[layer, 0], EPS)
        if chain.is_full_attention(layer):
            # (checked below through the GPU's own key input: the in-place key rows are outputs by now)
            want["fa_layer"] = layer
        else:
            conv = np.empty((rows.size, 10240), np.uint16)
            for i in range(rows.size):
                out, _ = orc.causal_conv1d_silu(window[i, 3:4], conv_w[layer], np.ascontiguousarray(window[i, :3].T))
                conv[i] = out[0]
            want["conv"] = conv
            want["q_l2"] = orc.l2_normalize_heads(conv[:, :2048].reshape(-1, 128), EPS, qs).reshape(rows.size, 2048)
            want["k_l2"] = orc.l2_normalize_heads(conv[:, 2048:4096].reshape(-1, 128), EPS, 1.0).reshape(rows.size, 2048)
            want["gdn_out"] = orc.rms_norm_rows(inp["gdn_core"].reshape(rows.size, 48, 128), gdn_w[layer], EPS,
                                                centered=False, gate=inp["gdn_z"].reshape(rows.size, 48, 128)
                                                ).reshape(rows.size, 6144)
        residual, want["normalized"] = orc.residual_add_rms_norm(residual, inp["proj_out"], norm_w[layer, 1], EPS)
    want["mlp"] = orc.silu_mul(inp["mlp_gate"], inp["mlp_up"])

    # ---- residual stream: eight roundings deep, bit-exact ------------------------------------------
    g.assert_bits_equal(take(final), residual, "final residual stream")
    # ---- last norm + NVFP4 --------------------------------------------------------------------------
    got_n = take(stack.normalized)
    g.assert_bf16_within(got_n, want["normalized"], 1, 0.98, "normalized rows")
    groups = rows // chain.CHUNK
    gs = stack.global_scales.cpu().numpy()
    # global scales: from the GPU's own normalised rows, whole groups (amax / 2688, or 1 for an all-zero group)
    n_all = stack.normalized.float().abs()
    n_all = torch.where(torch.isfinite(n_all), n_all, torch.zeros_like(n_all))
    pad = (-total) % chain.CHUNK
    amax = torch.nn.functional.pad(n_all.amax(dim=1), (0, pad)).reshape(-1, chain.CHUNK).amax(dim=1).cpu().numpy()
    want_gs = np.where(amax == 0, np.float32(1.0), amax.astype(np.float32) / np.float32(2688.0)).astype(np.float32)
    assert np.array_equal(gs.view(np.uint32), want_gs.view(np.uint32)), "global scales of the last norm"
    got_codes, got_scales = take(stack.codes), take(stack.scales)
    for grp in np.unique(groups):
        sel = groups == grp
        c, s = orc.nvfp4_quantize_with_scales(got_n[sel], gs[grp:grp + 1], 0)
        g.assert_bits_equal(got_codes[sel], c, f"codes, scale group {grp}")
        g.assert_bits_equal(got_scales[sel], s, f"block scales, scale group {grp}")
    # ---- GDN operators (layer 2 wrote them last) -------------------------------------------------------
    got_conv = take(stack.conv_out)
    g.assert_bf16_within(got_conv[:, 4096:], want["conv"][:, 4096:], 1, 0.98, "conv v channels")
    g.assert_reference_tolerance(got_conv[:, :2048], want["q_l2"], "conv -> L2 (q)")
    g.assert_reference_tolerance(got_conv[:, 2048:4096], want["k_l2"], "conv -> L2 (k)")
    worst, exact = g.ulp_report(got_conv[:, :4096], np.concatenate([want["q_l2"], want["k_l2"]], axis=1))
    assert worst <= 2 and exact > 0.97, (worst, exact)
    got_gdn = take(stack.gdn_out)
    g.assert_bf16_within(got_gdn, want["gdn_out"], 1, 0.98, "gated norm")
    # (the GDN global scales were overwritten by the later residual norms, which share the buffer: the
    # codes are checked for self-consistency with the block scales they were written with)
    # ---- full-attention operators (layer 3) -----------------------------------------------------------------
    layer = want["fa_layer"]
    q_norm = orc.rms_norm_rows(inp["q_gate"].reshape(rows.size, 24, 2, 256)[:, :, 0, :], q_w[layer], EPS)
    want_q = np.stack([orc.partial_rope(q_norm[i], cos[rows[i]], sin[rows[i]]) for i in range(rows.size)])
    got_q = take(stack.q_out).reshape(rows.size, 24, 256)
    g.assert_bf16_within(got_q[..., 64:], want_q[..., 64:], 1, 0.98, "q pass-through dims")
    g.assert_reference_tolerance(got_q, want_q, "q end to end", amplified=True)
    assert g.ulp_report(got_q[..., :64], want_q[..., :64])[1] > 0.97
    want_gate = inp["q_gate"].reshape(rows.size, 24, 2, 256)[:, :, 1, :].reshape(rows.size, 6144)
    g.assert_bits_equal(take(stack.gate_out), want_gate, "gate copy")
    g.assert_bf16_within(take(stack.attn_out), orc.sigmoid_gate(inp["attn_value"], want_gate), 1, 0.98, "sigmoid gate")
    # ---- MLP ----------------------------------------------------------------------------------------------
    g.assert_bf16_within(take(stack.mlp_out), want["mlp"], 1, 0.98, "SwiGLU")


def test_key_rows_of_the_chain_against_the_oracle(g):
    """The full-attention layer normalises and rotates the key rows IN PLACE, so the chain's key tensor is
    input and output at once; a copy taken before the step is the oracle's input."""
    total, layers = 4096, 4
    stack = chain.LayerStack(total, first_position=1000, seed=35, layers=layers, table_rows=4096)
    key_before = bits(stack.inputs["key"]).reshape(total, 4, 256)
    stack.enqueue_step(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    stack.check_error("chain under test")
    cos, sin = stack.cos.cpu().numpy(), stack.sin.cpu().numpy()  # the operator's own input tables
    k_norm = orc.rms_norm_rows(key_before, bits(stack.k_norm_w)[3], chain.EPS)
    want = np.stack([orc.partial_rope(k_norm[t], cos[1000 + t], sin[1000 + t]) for t in range(total)])
    got = bits(stack.inputs["key"]).reshape(total, 4, 256)
    g.assert_bf16_within(got[..., 64:], want[..., 64:], 1, 0.98, "k pass-through dims")
    g.assert_reference_tolerance(got, want, "k end to end", amplified=True)
    assert g.ulp_report(got[..., :64], want[..., :64])[1] > 0.97


def test_fp32_intermediates_within_1e_5_relative(g):
    """The FP32 building blocks of the kernels (inverse RMS, inverse L2 norm, SiLU, branch-stable sigmoid,
    exp(-|x|)) against the host reference's expressions evaluated in float64, relative error <= 1e-5
    wherever the exact value is a normal float (below that the absolute error is bounded instead)."""
    rng = np.random.default_rng(100000)
    TOL = 1e-5

    def run(function, x, p0=0.0, p1=0.0):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = g.empty_like_dev((x.size,), dtype=np.float32)
        g.capi.check("q3x_b200_debug_intermediate", g.Dev(x), x.size, function, p0, p1, out, None)
        g.sync()
        return out.get().astype(np.float64)

    def check(got, exact, what):
        exact = np.asarray(exact, dtype=np.float64)
        normal = np.abs(exact) >= 2.0 ** -126
        rel = np.abs(got[normal] - exact[normal]) / np.abs(exact[normal])
        assert rel.size and rel.max() <= TOL, f"{what}: relative error {rel.max():.3e}"
        assert np.all(np.abs(got[~normal] - exact[~normal]) <= 2.0 ** -126 * TOL * 8), f"{what}: subnormal range"

    # sums of squares as the kernels see them: 5120 / 256 / 128 elements of N(0, s^2), s from 1e-3 to 1e3
    scale = 10.0 ** rng.uniform(-3, 3, size=200_000)
    for width, eps in ((5120.0, 1e-6), (256.0, 1e-6), (128.0, 1e-6)):
        sums = (scale ** 2 * width * rng.uniform(0.5, 1.5, size=scale.size)).astype(np.float32)
        sums[:8] = [0.0, 1e-30, 1e-12, 1.0, 3.0e38, 1e20, 5120.0, 2.5e-7]
        s64 = sums.astype(np.float64)
        e32 = np.float64(np.float32(eps))
        check(run(0, sums, width, eps), 1.0 / np.sqrt(s64 / width + e32), f"inverse RMS, width {int(width)}")
        check(run(1, sums, 0.0, eps), 1.0 / np.sqrt(s64 + e32), "inverse L2 norm")
    # activations: dense in [-30, 30] plus the tails up to the largest bf16 magnitudes that matter
    x = np.concatenate([rng.uniform(-30, 30, 400_000), rng.uniform(-87, -30, 50_000), rng.uniform(30, 90, 50_000),
                        rng.standard_normal(200_000), [0.0, -0.0, 1e-20, -1e-20, 88.0, -86.9]]).astype(np.float32)
    x64 = x.astype(np.float64)
    sig = np.where(x64 >= 0, 1.0 / (1.0 + np.exp(-x64)), np.exp(x64) / (1.0 + np.exp(x64)))
    check(run(2, x), x64 / (1.0 + np.exp(-x64)), "silu")
    check(run(3, x), x64 / (1.0 + np.exp(-x64)), "silu (SwiGLU form)")
    check(run(4, x), sig, "stable sigmoid")
    check(run(5, x), np.exp(-np.abs(x64)), "exp(-|x|)")
