"""GPU test of the bulk causal GQA attention of a tile of tokens with the sigmoid output gate
(q3x_b200_gqa_attention_prefill_sigmoid_gate), through the C ABI, against the oracle's attention (pinned to the
reference's gqa_attention_reference_cpu + sigmoid_gate_reference_cpu) applied token by token: token t of the tile
sees cache positions 0 .. first_position + t.

Tolerance.  The host reference keeps the softmax probabilities in FP32; the kernel hands each one to the tensor
cores as two bf16 operands (16 significant bits), so what separates the two is the order of the FP32 sums: the
batch-one kernel's rule (ulps + a rounding-level floor + an exact-match quota) and the reference's acceptance rule
max(2e-3, 8e-3 |e|) (tests/decode_ops_cuda_test.cu:432-450) as the hard bound."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import fixtures as fx

pytestmark = pytest.mark.gpu
SCALE = 0.0625


@pytest.fixture(scope="module")
def g():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    return gpu_util


def expected(q, kc, vc, gate, first):
    rows = []
    for t in range(q.shape[0]):
        length = first + t + 1
        out, _ = orc.gqa_attention(q[t], kc[:length], vc[:length], SCALE, gate=None if gate is None else gate[t])
        rows.append(out)
    return np.stack(rows)


@pytest.mark.parametrize("tokens,first,gated,sharp", [(2, 0, True, 1.0), (16, 0, False, 1.0), (40, 0, True, 1.0),
                                                       (37, 100, True, 1.0), (130, 63, True, 3.0), (512, 0, True, 1.0),
                                                       (200, 512, True, 1.0), (64, 1000, False, 3.0),
                                                       # (tiles longer than the reference's 512)
                                                       (1100, 0, True, 1.0), (1030, 77, False, 3.0)])
def test_prefill_attention_matches_the_per_token_reference(g, tokens, first, gated, sharp):
    rng = np.random.default_rng([tokens, first, int(gated), 111])
    length = first + tokens
    q = fx.normal_bf16(rng, (tokens, 24, 256), sharp)
    kc, vc = fx.normal_bf16(rng, (length, 4, 256)), fx.normal_bf16(rng, (length, 4, 256))
    gate = fx.normal_bf16(rng, (tokens, 24, 256), 2.0) if gated else None
    out = g.empty_like_dev((tokens, 24, 256))
    g.capi.check("q3x_b200_gqa_attention_prefill_sigmoid_gate", g.Dev(q), g.Dev(kc), g.Dev(vc),
                 g.Dev(gate) if gated else None, first, tokens, SCALE, out, None)
    g.sync()
    assert out.guards_intact()
    want = expected(q, kc, vc, gate, first)
    got = out.get()
    # as for the batch-one kernel: one rounding of an FP32 weighted average summed in another order (1 ulp plus a
    # rounding-level fraction of the terms' magnitude); the gate multiplies the ROUNDED attention, so a 1-ulp
    # difference there passes through (up to 3 ulps of the smaller gated value)
    g.assert_sum_within(got, want, 3 if gated else 1, 1e-5, 0.98, "prefill attention")
    # The reference's rule is a hard bound for the attention itself.  Behind the gate it is a two-rounding chain: a
    # 1-ulp difference of the rounded attention, scaled by sigmoid(gate) and rounded again, can come out as 2 ulps
    # of a value at the bottom of its binade (3.9e-3 at 0.48 against 8e-3 x 0.48 = 3.87e-3; about one element in a
    # million): there the rule is the quota form (at most 2 per 100 000 outside it, two ulps of the row as the bound).
    g.assert_reference_tolerance(got, want, "prefill attention", amplified=gated)


def test_prefill_attention_of_a_long_tile_on_sampled_tokens(g):
    """A 4133-token tile appended at position 50 (33 CTAs of 128 tokens on the tcgen05 path, the last one holding 37;
    on the mma.sync path this length takes the wide CTA shape), checked against the per-token oracle on sampled tokens,
    block edges and the tile's two ends -- on both paths."""
    rng = np.random.default_rng(119)
    tokens, first = 4133, 50
    length = first + tokens
    q = fx.normal_bf16(rng, (tokens, 24, 256))
    kc, vc = fx.normal_bf16(rng, (length, 4, 256)), fx.normal_bf16(rng, (length, 4, 256))
    gate = fx.normal_bf16(rng, (tokens, 24, 256), 2.0)
    picks = sorted(set([0, 1, 15, 16, 127, 128, 129, 2047, 2048, 4095, 4096, 4111, 4112, 4127, 4128, 4131, 4132]) |
                   set(int(t) for t in rng.choice(tokens, size=48, replace=False)))
    want = np.stack([orc.gqa_attention(q[t], kc[:first + t + 1], vc[:first + t + 1], SCALE, gate=gate[t])[0] for t in picks])
    d_q, d_k, d_v, d_g = g.Dev(q), g.Dev(kc), g.Dev(vc), g.Dev(gate)
    for path in (1, 0):
        out = g.empty_like_dev((tokens, 24, 256))
        g.capi.check("q3x_b200_gqa_prefill_select_path", path)
        try:
            g.capi.check("q3x_b200_gqa_attention_prefill_sigmoid_gate", d_q, d_k, d_v, d_g, first, tokens, SCALE, out, None)
            g.sync()
        finally:
            g.capi.check("q3x_b200_gqa_prefill_select_path", 1)
        assert out.guards_intact()
        got = out.get()[picks]
        g.assert_sum_within(got, want, 3, 1e-5, 0.98, f"prefill attention, long tile, path {path}")
        g.assert_reference_tolerance(got, want, f"prefill attention, long tile, path {path}", amplified=True)
        assert bool(np.isfinite(orc.bf16_decode(out.get())).all())
    assert g.capi.lib().q3x_b200_gqa_prefill_tcgen05_error() == 0


@pytest.mark.parametrize("path", [1, 0])
def test_prefill_attention_with_rising_scores(g, path):
    """Scores that climb by about 30 (in units of the exponent, log2) per 64-key tile: the running maximum of every row
    keeps moving, which on the tcgen05 path (1) makes the reference maximum jump and the accumulator in tensor memory
    be rescaled several times per row, and on the mma.sync path (0) exercises the per-tile correction.  Both against the
    per-token oracle; and the tcgen05 path's error word stays clear."""
    rng = np.random.default_rng(121)
    tokens, first = 300, 40
    length = first + tokens
    q = orc.bf16_encode(np.ones((tokens, 24, 256), np.float32) + 0.05 * rng.standard_normal((tokens, 24, 256)).astype(np.float32))
    ramp = (np.arange(length, dtype=np.float32) * 0.02)[:, None, None]           # q . k grows by 5.1 per key
    kc = orc.bf16_encode(ramp * np.ones((length, 4, 256), np.float32) + 0.05 * rng.standard_normal((length, 4, 256)).astype(np.float32))
    vc = fx.normal_bf16(rng, (length, 4, 256))
    gate = fx.normal_bf16(rng, (tokens, 24, 256), 2.0)
    out = g.empty_like_dev((tokens, 24, 256))
    g.capi.check("q3x_b200_gqa_prefill_select_path", path)
    try:
        g.capi.check("q3x_b200_gqa_attention_prefill_sigmoid_gate", g.Dev(q), g.Dev(kc), g.Dev(vc), g.Dev(gate), first, tokens,
                     SCALE, out, None)
        g.sync()
    finally:
        g.capi.check("q3x_b200_gqa_prefill_select_path", 1)
    assert out.guards_intact()
    assert g.capi.lib().q3x_b200_gqa_prefill_tcgen05_error() == 0
    want = expected(q, kc, vc, gate, first)
    g.assert_sum_within(out.get(), want, 3, 1e-5, 0.98, "prefill attention, rising scores")
    g.assert_reference_tolerance(out.get(), want, "prefill attention, rising scores", amplified=True)


def test_both_prefill_attention_paths_agree(g):
    """The mma.sync path on the inputs of the first test's largest case, against the tcgen05 path (the default, which
    every other test here runs): same operands, sums in another order."""
    rng = np.random.default_rng(122)
    tokens, first = 700, 100
    length = first + tokens
    q = fx.normal_bf16(rng, (tokens, 24, 256))
    kc, vc = fx.normal_bf16(rng, (length, 4, 256)), fx.normal_bf16(rng, (length, 4, 256))
    gate = fx.normal_bf16(rng, (tokens, 24, 256), 2.0)
    outs = []
    for path in (1, 0):
        out = g.empty_like_dev((tokens, 24, 256))
        g.capi.check("q3x_b200_gqa_prefill_select_path", path)
        try:
            g.capi.check("q3x_b200_gqa_attention_prefill_sigmoid_gate", g.Dev(q), g.Dev(kc), g.Dev(vc), g.Dev(gate), first,
                         tokens, SCALE, out, None)
            g.sync()
        finally:
            g.capi.check("q3x_b200_gqa_prefill_select_path", 1)
        outs.append(out.get())
    assert g.capi.lib().q3x_b200_gqa_prefill_tcgen05_error() == 0
    assert np.mean(outs[0] == outs[1]) > 0.99
    # (both round the same FP32 weighted averages summed in another order: one ulp apart where they differ, two behind
    # the gate at the bottom of a binade -- the rule of the oracle comparison above, one path standing in for the oracle)
    g.assert_sum_within(outs[0], outs[1], 3, 1e-5, 0.99, "tcgen05 against mma.sync")
    g.assert_reference_tolerance(outs[0], outs[1], "tcgen05 against mma.sync", amplified=True)
    assert g.capi.call("q3x_b200_gqa_prefill_select_path", 3) == 1


def test_prefill_attention_equals_decode_attention_on_its_last_token(g):
    """The tile's last token sees the whole cache: the same query through the batch-one kernel."""
    rng = np.random.default_rng(112)
    tokens, first = 48, 300
    length = first + tokens
    q = fx.normal_bf16(rng, (tokens, 24, 256))
    kc, vc = fx.normal_bf16(rng, (length, 4, 256)), fx.normal_bf16(rng, (length, 4, 256))
    gate = fx.normal_bf16(rng, (tokens, 24, 256), 2.0)
    d_k, d_v = g.Dev(kc), g.Dev(vc)
    out = g.empty_like_dev((tokens, 24, 256))
    g.capi.check("q3x_b200_gqa_attention_prefill_sigmoid_gate", g.Dev(q), d_k, d_v, g.Dev(gate), first, tokens, SCALE, out, None)
    words = g.capi.lib().q3x_b200_gqa_decode_workspace_floats(length)
    ws = g.empty_like_dev((words,), dtype=np.float32)
    one = g.empty_like_dev((24, 256))
    g.capi.check("q3x_b200_gqa_attention_decode_sigmoid_gate", g.Dev(q[-1]), d_k, d_v, length, SCALE, ws, words,
                 g.Dev(gate[-1]), one, None)
    g.sync()
    a = orc.bf16_decode(out.get()[-1]).astype(np.float64)
    b = orc.bf16_decode(one.get()).astype(np.float64)
    assert np.all(np.abs(a - b) <= np.maximum(2.0e-3, 8.0e-3 * np.abs(b)))


def test_prefill_attention_rejections(g):
    inv, fake = g.capi.CUDA_ERROR_INVALID_VALUE, 0x10000000
    call = lambda **kw: g.capi.call("q3x_b200_gqa_attention_prefill_sigmoid_gate", kw.get("q", fake), fake + (1 << 26),
                                    fake + (2 << 26), fake + (3 << 26), 0, kw.get("t", 16), kw.get("s", SCALE),
                                    kw.get("out", fake + (4 << 26)), None)
    assert call(q=None) == inv
    assert call(s=0.0) == inv
    assert call(out=fake) == inv
    assert call(t=0) == 0
