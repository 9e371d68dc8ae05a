"""Generates tests/golden/reference_core_ops.npz: inputs and outputs of the REFERENCE's own host ops for the
operators between the fused layer ops (gated-delta-net recurrence step, softmax, GQA attention, the bf16 and
NVFP4 batch-one GEMVs), produced by calling oracle/_ref/libq3x_ref.so (the reference's sources compiled from a
reference checkout by oracle/Makefile).  Run where a reference checkout exists:

    python tests/golden/make_golden_core.py

The fixtures travel with the repository; the tests that use them need no reference checkout.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as orc  # noqa: E402
from tests import fixtures as fx  # noqa: E402

u16p, u8p, f32p = C.POINTER(C.c_uint16), C.POINTER(C.c_uint8), C.POINTER(C.c_float)


def p(a, ty=u16p):
    return a.ctypes.data_as(ty)


def structured_state():
    return fx.structured_bf16(48 * 128 * 128, 251, 125, 1000).reshape(48, 128, 128)


def gdn_inputs(rng, tokens):
    conv = fx.normal_bf16(rng, (tokens, 10240))
    a, b = fx.normal_bf16(rng, (tokens, 48)), fx.normal_bf16(rng, (tokens, 48))
    A_log = orc.bf16_encode(rng.uniform(-4.0, 1.5, 48).astype(np.float32))
    dt_bias = orc.bf16_encode(rng.uniform(-3.0, 3.0, 48).astype(np.float32))
    # the state is 1.5 MB: a structured pattern that the test rebuilds instead of a stored random tensor
    state = structured_state()
    return conv, a, b, A_log, dt_bias, state


def main():
    orc.build()
    ref = orc.ref_lib()
    if ref is None:
        raise SystemExit("oracle/_ref is not built: a reference checkout is needed to generate fixtures")
    rng = np.random.default_rng(20260125)
    g = {}
    # three recurrence steps through the single-token reference op, state carried in place
    conv, a, b, A_log, dt_bias, state = gdn_inputs(rng, 3)
    st = state.copy()
    outs = np.empty((3, 6144), np.uint16)
    for t in range(3):
        o = np.empty(6144, np.uint16)
        assert ref.gdn_update(p(np.ascontiguousarray(conv[t])), p(np.ascontiguousarray(a[t])),
                              p(np.ascontiguousarray(b[t])), p(A_log), p(dt_bias), p(st), p(st), 1e-6, p(o)) == 0
        outs[t] = o
    # the state is 1.5 MB: keep heads 0, 17 and 47 of input and output
    keep = [0, 17, 47]
    g.update(gdn_conv=conv, gdn_a=a, gdn_b=b, gdn_A_log=A_log, gdn_dt_bias=dt_bias, gdn_out_want=outs, gdn_state_heads=np.array(keep), gdn_state_want=st[keep])
    # softmax
    x = (rng.standard_normal((5, 37)) * 4).astype(np.float32)
    x[1, 3] = 80.0
    x[2, :] = -1e30
    y = np.empty_like(x)
    assert ref.softmax(p(x, f32p), 5, 37, p(y, f32p)) == 0
    g.update(softmax_x=x, softmax_want=y)
    # GQA attention 24 / 4 / 256 over 70 positions
    q = fx.normal_bf16(rng, (24, 256))
    kc, vc = fx.normal_bf16(rng, (70, 4, 256)), fx.normal_bf16(rng, (70, 4, 256))
    scratch = np.empty((24, 70), np.float32)
    out = np.empty((24, 256), np.uint16)
    assert ref.gqa(p(q), p(kc), p(vc), 24, 4, 70, 256, 0.0625, p(scratch, f32p), scratch.size, p(out)) == 0
    g.update(gqa_q=q, gqa_k=kc, gqa_v=vc, gqa_probs_want=scratch.copy(), gqa_out_want=out)
    # GEMVs
    w = fx.normal_bf16(rng, (19, 320), 0.05)
    xv = fx.normal_bf16(rng, (320,))
    o = np.empty(19, np.float32)
    assert ref.bf16_gemv(p(w), p(xv), 19, 320, p(o, f32p)) == 0
    g.update(gemv_w=w, gemv_x=xv, gemv_want=o.copy())
    packed = rng.integers(0, 256, size=(19, 160), dtype=np.uint8)
    scales = rng.integers(0x20, 0x50, size=(19, 20), dtype=np.uint8)
    o2 = np.empty(19, np.float32)
    assert ref.nvfp4_gemv(p(packed, u8p), p(scales, u8p), 0.0123, p(xv), 19, 320, p(o2, f32p)) == 0
    g.update(nvfp4_gemv_packed=packed, nvfp4_gemv_scales=scales, nvfp4_gemv_scale2=np.array([0.0123], np.float32),
             nvfp4_gemv_want=o2)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_core_ops.npz")
    np.savez_compressed(path, **g)
    print("wrote", path, os.path.getsize(path), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
