"""Helpers of the GPU parity tests: device buffers with canary guards, bf16 comparisons in ulps,
and the loader of the C-ABI library.  Everything on the device goes through ``capi`` (ctypes)."""
import importlib

import numpy as np
import torch

from oracle import oracle as orc

pkg = importlib.import_module("qwen3x-orin_b200")
capi = pkg.capi

GUARD = 64  # elements of canary on both sides of every guarded buffer
CANARY16 = 0xC0DE
CANARY8 = 0xA5


class Dev:
    """A device buffer holding a numpy array, surrounded by canaries.  ``t`` is the payload view."""

    def __init__(self, array, misalign=0):
        array = np.ascontiguousarray(array)
        self.dtype = array.dtype
        self.shape = array.shape
        n = array.size
        if array.dtype == np.uint16:
            carrier, canary = torch.int16, np.array(CANARY16, dtype=np.uint16).view(np.int16).item()
        elif array.dtype == np.uint8:
            carrier, canary = torch.uint8, CANARY8
        elif array.dtype == np.float32:
            carrier, canary = torch.float32, -12345.5
        elif array.dtype == np.uint32:
            carrier, canary = torch.int32, 0x5A5A5A5A
        else:
            raise TypeError(array.dtype)
        self.canary = canary
        # 16-byte aligned payload start (plus an optional deliberate misalignment in elements)
        item = array.dtype.itemsize
        pad = (16 // item) * ((GUARD * item + 15) // 16) + misalign
        self.pad = pad
        self.full = torch.full((pad + n + GUARD,), canary, dtype=carrier, device="cuda")
        self.t = self.full[pad:pad + n]
        if n:
            signed = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32}.get(array.dtype, array.dtype)
            self.t.copy_(torch.from_numpy(array.reshape(-1).view(signed).copy()))

    def data_ptr(self):
        return self.t.data_ptr()

    def ptr_at(self, element):
        return self.t.data_ptr() + element * self.dtype.itemsize

    def get(self):
        host = self.t.cpu().numpy()
        return host.view(self.dtype).reshape(self.shape).copy()

    def guards_intact(self):
        head = self.full[:self.pad]
        tail = self.full[self.pad + self.t.numel():]
        return bool((head == self.canary).all().item() and (tail == self.canary).all().item())


def empty_like_dev(shape, dtype=np.uint16, misalign=0, fill=None):
    a = np.zeros(shape, dtype=dtype)
    if fill is not None:
        a[...] = fill
    return Dev(a, misalign)


def scratch_for(rows, rows_per_scale, fill=0):
    """The caller-owned scratch of the NVFP4 entry points, zeroed once as the contract asks (every call
    leaves it zero again; the last word is the sticky error flag)."""
    words = capi.lib().q3x_b200_nvfp4_scratch_words(rows, rows_per_scale)
    return empty_like_dev((words,), dtype=np.uint32, fill=0)


def assert_scratch_clean(scratch, what=""):
    """After any NVFP4 call: every scratch word is zero again and no bounded wait gave up."""
    words = scratch.get()
    assert words[-1] == 0, f"{what}: a bounded device-side wait gave up (error word {words[-1]:#x})"
    assert not words.any(), f"{what}: the call left {int(np.count_nonzero(words))} scratch words non-zero"


def sync():
    torch.cuda.synchronize()


def ulp_report(got, want):
    """(max ulp distance, fraction of bit-exact elements); NaN matches NaN."""
    d = orc.bf16_ulp_distance(got, want)
    nan_g, nan_w = orc.bf16_is_nan(got), orc.bf16_is_nan(want)
    exact = (np.asarray(got) == np.asarray(want)) | (nan_g & nan_w)
    return int(d.max()) if d.size else 0, float(exact.mean()) if d.size else 1.0


def assert_bf16_within(got, want, max_ulp=1, min_exact=0.0, what=""):
    """north_star tolerance for bf16 outputs: within 1 bf16 ulp of the host reference op."""
    worst, exact = ulp_report(got, want)
    assert worst <= max_ulp, f"{what}: max distance {worst} ulp (allowed {max_ulp}), exact fraction {exact:.6f}"
    assert exact >= min_exact, f"{what}: only {exact:.6f} of the elements are bit-exact"
    return worst, exact


def assert_reference_tolerance(got, want, what="", amplified=False):
    """The reference's own acceptance rule for a bf16 result (expect_bf16_match,
    tests/decode_ops_cuda_test.cu:432-450): NaN matches NaN, an infinity matches the same infinity, every
    other value within max(2e-3, 8e-3 * |expected|).

    It is a hard bound for chains whose second stage only scales (conv -> L2 norm).  With ``amplified`` (the
    rotated dims of norm -> RoPE) it cannot be one for ANY implementation whose first rounding is not
    bit-identical to the host's: the rotation subtracts two products, so a 1-ulp difference of an operand
    (the stage-wise tolerance) survives at the operand's magnitude while the result may be smaller.  There
    the rule is applied as a quota -- at most 2 elements in 100 000 outside it -- and the hard bound is the
    one arithmetic gives: two ulps at the largest magnitude of the element's row (the rotation's operands)."""
    a = orc.bf16_decode(np.asarray(got)).astype(np.float64)
    e = orc.bf16_decode(np.asarray(want)).astype(np.float64)
    row_scale = np.broadcast_to(np.nanmax(np.where(np.isfinite(e), np.abs(e), 0.0), axis=-1, keepdims=True), e.shape)
    a, e, row_scale = a.reshape(-1), e.reshape(-1), row_scale.reshape(-1)
    nan_e, inf_e = np.isnan(e), np.isinf(e)
    assert np.array_equal(np.isnan(a), nan_e), f"{what}: NaN classification differs"
    assert np.array_equal(a[inf_e], e[inf_e]), f"{what}: infinity classification differs"
    fin = ~(nan_e | inf_e)
    tol = np.maximum(2.0e-3, np.abs(e[fin]) * 8.0e-3)
    err = np.abs(a[fin] - e[fin])
    bad = np.nonzero(err > tol)[0]
    allowed = int(np.ceil(2.0e-5 * err.size)) if amplified else 0
    assert bad.size <= allowed, (f"{what}: {bad.size} of {err.size} elements beyond max(2e-3, 8e-3|e|) ({allowed} allowed); "
                                 f"worst {err[bad].max():.3e} at expected {e[fin][bad[np.argmax(err[bad])]]:.6g}")
    if bad.size:
        # two bf16 ulps AT the row's largest magnitude m: 2 * 2^(floor(log2 m) - 7), which lies between 2^-7 m and 2^-6 m
        scale = np.maximum(row_scale[fin][bad], 2.0 ** -120)
        hard = 2.0 * 2.0 ** (np.floor(np.log2(scale)) - 7.0)
        assert np.all(err[bad] <= hard), f"{what}: an element differs by more than two ulps of its row's magnitude"


def assert_sum_within(got, want, ulps, floor, min_exact, what=""):
    """Tolerance for a bf16 result that is the rounding of a long FP32 sum with cancellation (an attention
    output, a recurrence output): the FP32 sum differs from the host's by a rounding-level fraction of the sum
    of its terms' MAGNITUDES, which is many ulps of the result wherever the terms cancel.  So: within `ulps`
    bf16 ulps of the expected value plus an absolute `floor` (a few 1e-6 of the terms' magnitude), and a
    quota of bit-exact elements."""
    g_bits, w_bits = np.asarray(got).reshape(-1), np.asarray(want).reshape(-1)
    a, e = orc.bf16_decode(g_bits).astype(np.float64), orc.bf16_decode(w_bits).astype(np.float64)
    assert np.array_equal(np.isnan(a), np.isnan(e)), f"{what}: NaN classification differs"
    fin = np.isfinite(e)
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(e[fin]), 2.0 ** -126))) - 7)
    err = np.abs(a[fin] - e[fin])
    worst = np.max(err - (ulps * ulp + floor)) if err.size else 0.0
    assert worst <= 0, f"{what}: an element is {worst:.3e} beyond {ulps} ulp + {floor:g}"
    exact = float(np.mean(g_bits == w_bits)) if g_bits.size else 1.0
    assert exact >= min_exact, f"{what}: only {exact:.6f} of the elements are bit-exact"


def assert_bits_equal(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    bad = np.nonzero(got.reshape(-1) != want.reshape(-1))[0]
    assert bad.size == 0, f"{what}: {bad.size} mismatching elements, first at {bad[:5]}"
