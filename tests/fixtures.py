"""Seeded input builders shared by the CPU and GPU parity tests.

``special_bf16`` collects the bit patterns the reference's own tests probe
(tests/decode_ops_host_test.cpp:456-478 and the non-finite fixture of
tests/decode_ops_cuda_test.cu:1771-1826): signed zeros, infinities, quiet and tiny-payload
NaNs, subnormals, the largest finite value and values next to rounding midpoints.
"""
import numpy as np

from oracle import oracle as orc


def normal_bf16(rng, shape, std=1.0):
    return orc.bf16_encode((rng.standard_normal(shape) * std).astype(np.float32))


def special_bf16():
    return np.array(
        [0x0000, 0x8000, 0x7F80, 0xFF80, 0x7FC0, 0xFFC0, 0x7F81, 0xFFA5, 0x0001, 0x8001, 0x007F,
         0x0080, 0x7F7F, 0xFF7F, 0x3F80, 0xBF80, 0x3F81, 0x4000, 0x40A0, 0x3E80, 0x3F40, 0x3FA0,
         0x3FE0, 0x4020, 0x4060, 0x42B0, 0xC2B0, 0x4300, 0x4580],
        dtype=np.uint16)


def sprinkle_specials(rng, bits, fraction=0.01):
    """Overwrite a random ``fraction`` of ``bits`` (in place) with special bit patterns."""
    flat = bits.reshape(-1)
    count = max(1, int(flat.size * fraction))
    where = rng.choice(flat.size, size=count, replace=False)
    sp = special_bf16()
    flat[where] = sp[rng.integers(0, sp.size, size=count)]
    return bits


def structured_bf16(count, modulus, offset, divisor):
    """The ``(i*k % m - o) / d`` style of deterministic fixture the reference's tests use."""
    i = np.arange(count, dtype=np.int64)
    return orc.bf16_encode(((i % modulus) - offset).astype(np.float32) / np.float32(divisor))


def xorshift_bf16(count, seed=0x9E3779B9, scale=4.0):
    """xorshift32 stream mapped to [-scale, scale): the "random-like" fixture family."""
    out = np.empty(count, dtype=np.float32)
    s = np.uint32(seed)
    with np.errstate(over="ignore"):
        for i in range(count):
            s ^= np.uint32(s << np.uint32(13))
            s ^= np.uint32(s >> np.uint32(17))
            s ^= np.uint32(s << np.uint32(5))
            out[i] = (float(s) / 4294967296.0 * 2.0 - 1.0) * scale
    return orc.bf16_encode(out)
