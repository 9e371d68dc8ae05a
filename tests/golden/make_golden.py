"""Generates tests/golden/reference_ops.npz from the reference project's own host reference ops.

Run in a container that holds a reference checkout:

    make -C oracle ref && python tests/golden/make_golden.py

Every array named ``*_want`` is the output of a reference function (compiled unmodified into
oracle/_ref/libq3x_ref.so) on the seeded inputs stored beside it, so the fixtures pin both the C
restatement (CPU tests) and the CUDA path (GPU tests) on machines without a reference checkout.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402
from tests import fixtures as fx  # noqa: E402

u16p = C.POINTER(C.c_uint16)
f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)
EPS = 1e-6


def p(a, ty=u16p):
    return a.ctypes.data_as(ty)


def main():
    orc.build()
    ref = orc.ref_lib()
    assert ref is not None, "oracle/_ref/libq3x_ref.so is missing: run `make -C oracle ref`"
    rng = np.random.default_rng(20261125)
    g = {}

    # residual add + centred RMSNorm, 6 rows of 5120 (one row carries special values)
    left = fx.normal_bf16(rng, (6, 5120))
    right = fx.normal_bf16(rng, (6, 5120))
    fx.sprinkle_specials(rng, left[5:], 0.002)
    w = fx.normal_bf16(rng, (5120,), 0.02)
    res = np.empty_like(left)
    nrm = np.empty_like(left)
    assert ref.residual_add(p(left), p(right), left.size, p(res)) == 0
    assert ref.head_centered(p(res), p(w), 6, 5120, EPS, p(nrm)) == 0
    g.update(rn_left=left, rn_right=right, rn_weight=w, rn_residual_want=res, rn_normalized_want=nrm)

    # pointwise ops on 777 elements with specials
    a = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (777,), 2.0), 0.03)
    b = fx.sprinkle_specials(rng, fx.normal_bf16(rng, (777,), 2.0), 0.03)
    for name, fn in (("residual", ref.residual_add), ("silu_mul", ref.silu_mul), ("sigmoid_gate", ref.sigmoid_gate)):
        out = np.empty_like(a)
        assert fn(p(a), p(b), 777, p(out)) == 0
        g[f"pw_{name}_want"] = out
    g.update(pw_a=a, pw_b=b)

    # head norms: q/k (centred, 256) and GDN output (plain, 128, SiLU gate)
    x = fx.normal_bf16(rng, (28, 256))
    hw = fx.normal_bf16(rng, (256,), 0.02)
    out = np.empty_like(x)
    assert ref.head_centered(p(x), p(hw), 28, 256, EPS, p(out)) == 0
    g.update(hn_x=x, hn_w=hw, hn_centered_want=out.copy())
    x = fx.normal_bf16(rng, (48, 128))
    z = fx.normal_bf16(rng, (48, 128))
    gw = orc.bf16_encode((0.75 + rng.random(128) * 0.5).astype(np.float32))
    out = np.empty_like(x)
    assert ref.head_plain_gate(p(x), p(gw), p(z), 48, 128, EPS, p(out)) == 0
    g.update(gn_x=x, gn_z=z, gn_w=gw, gn_want=out.copy())
    out2 = np.empty_like(x)
    assert ref.head_plain(p(x), p(gw), 48, 128, EPS, p(out2)) == 0
    g.update(gn_plain_want=out2)

    # L2 norm 16x128 and 5x127
    for tag, shape in (("a", (16, 128)), ("b", (5, 127))):
        x = fx.normal_bf16(rng, shape)
        out = np.empty_like(x)
        assert ref.l2(p(x), shape[0], shape[1], EPS, p(out)) == 0
        g[f"l2{tag}_x"] = x
        g[f"l2{tag}_want"] = out

    # RoPE at position 4096 and split
    cos, sin = orc.rope_tables(4096, 1)
    x = fx.normal_bf16(rng, (28, 256))
    out = np.empty_like(x)
    assert ref.rope(p(x), p(cos, f32p), p(sin, f32p), 28, p(out)) == 0
    g.update(rope_x=x, rope_cos=cos, rope_sin=sin, rope_want=out)
    qg = fx.normal_bf16(rng, (24, 2, 256))
    q = np.empty(24 * 256, dtype=np.uint16)
    gate = np.empty(24 * 256, dtype=np.uint16)
    assert ref.split(p(qg), 24, 256, p(q), p(gate)) == 0
    g.update(split_in=qg, split_q_want=q, split_gate_want=gate)

    # causal conv: 4 tokens through the single-token reference with non-zero history
    raw = fx.normal_bf16(rng, (4, 10240))
    cw = fx.normal_bf16(rng, (10240, 4), 0.5)
    hist = fx.normal_bf16(rng, (10240, 3))
    h = hist.copy()
    out = np.empty_like(raw)
    for t in range(4):
        row = np.ascontiguousarray(raw[t])
        o = np.empty(10240, dtype=np.uint16)
        assert ref.conv(p(row), p(cw), p(h), p(o)) == 0
        out[t] = o
    g.update(conv_raw=raw, conv_w=cw, conv_hist=hist, conv_want=out, conv_hist_want=h)

    # embedding: 5x7 table of the reference's own test, every row
    table = orc.bf16_encode(np.arange(35, dtype=np.float32) * np.float32(0.125) - np.float32(2.0)).reshape(5, 7)
    rows = np.empty((5, 7), dtype=np.uint16)
    for t in range(5):
        o = np.empty(7, dtype=np.uint16)
        assert ref.embedding(p(table), 5, 7, t, p(o)) == 0
        rows[t] = o
    g.update(emb_table=table, emb_want=rows)

    # format tables and the E4M3 quantiser observed through the static W8A8 GEMV
    g["e2m1_table"] = np.array([ref.decode_e2m1(i) for i in range(16)], dtype=np.float32)
    g["e4m3_table"] = np.array([ref.decode_e4m3(i) for i in range(256)], dtype=np.float32)
    probe = np.arange(0, 65536, 1, dtype=np.uint32).astype(np.uint16)
    vals = np.zeros(65536, dtype=np.float32)
    o = C.c_float()
    for i, bits in enumerate(probe.tolist()):
        if (bits & 0x7FFF) > 0x7F80:
            vals[i] = np.nan
            continue
        assert ref.e4m3_value(bits, 1.0, C.byref(o)) == 0
        vals[i] = o.value
    g["e4m3_quantised_of_every_bf16"] = vals

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_ops.npz")
    np.savez_compressed(path, **g)
    print("wrote", path, os.path.getsize(path), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
