"""CPU check of the softmax scheme of the tcgen05 prefill attention (gqa_prefill.cu): probabilities are taken against a
REFERENCE maximum that moves only when a 64-key tile exceeds it by more than 2^16 in the exponent's scale (then the
accumulator and the row sum are rescaled), each probability meets V as two bf16 operands (its rounding and the
rounding of the remainder), the row sum takes the probabilities unrounded.  Restated in numpy and compared with the
plain softmax-weighted average in float64: the scheme is the same function up to the two-operand rounding (2^-16
relative per probability), whatever the scores do -- flat, sharp, rising by many powers of two per tile, falling."""
import numpy as np
import pytest

TILE, THRESHOLD = 64, 16.0


def to_bf16(x):
    """Round-to-nearest-even float32 -> bf16, returned as float64 values."""
    bits = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64)


def lazy_attention_row(scores, values, scale_log2e):
    """One query row: scores [keys] (already masked to the visible keys), values [keys, dims]."""
    reference, row_sum = -np.inf, 0.0
    acc = np.zeros(values.shape[1])
    moves = 0
    for start in range(0, scores.size, TILE):
        s, v = scores[start:start + TILE], values[start:start + TILE]
        tile_max = s.max()
        if reference == -np.inf:
            reference = tile_max
        elif (tile_max - reference) * scale_log2e > THRESHOLD:
            factor = np.exp2((reference - tile_max) * scale_log2e)
            acc *= factor
            row_sum *= factor
            reference = tile_max
            moves += 1
        p = np.exp2((s - reference) * scale_log2e).astype(np.float32).astype(np.float64)
        row_sum += p.sum()
        hi = to_bf16(p)
        lo = to_bf16(p - hi)
        acc += (hi + lo) @ v
    return acc / row_sum, moves


@pytest.mark.parametrize("kind", ["flat", "sharp", "rising", "falling", "spike_late"])
def test_lazy_reference_maximum_and_two_operand_probabilities(kind):
    rng = np.random.default_rng([191, ["flat", "sharp", "rising", "falling", "spike_late"].index(kind)])
    keys, dims, scale_log2e = 1000, 32, 0.0625 * 1.4426950408889634
    values = to_bf16(rng.standard_normal((keys, dims)))
    scores = {
        "flat": rng.standard_normal(keys) * 10.0,
        "sharp": rng.standard_normal(keys) * 150.0,
        "rising": np.arange(keys) * 5.0 + rng.standard_normal(keys),          # 2^29 per tile
        "falling": -np.arange(keys) * 5.0 + rng.standard_normal(keys),
        "spike_late": np.where(np.arange(keys) == 777, 4000.0, rng.standard_normal(keys) * 10.0),
    }[kind]
    got, moves = lazy_attention_row(scores, values, scale_log2e)
    weights = np.exp2((scores - scores.max()) * scale_log2e)
    want = (weights @ values) / weights.sum()
    magnitude = (weights @ np.abs(values)) / weights.sum()
    assert np.all(np.abs(got - want) <= 2.0 ** -15 * magnitude + 1e-30), np.abs(got - want).max()
    if kind in ("rising", "spike_late"):
        assert moves >= 1, "this case is meant to move the reference maximum"
    if kind in ("flat", "falling"):
        assert moves == 0
