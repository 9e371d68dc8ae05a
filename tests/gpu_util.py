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


def assert_reference_tolerance(got, want, what=""):
    """The reference's own acceptance rule for a bf16 result (expect_bf16_match,
    tests/decode_ops_cuda_test.cu:432-450): NaN matches NaN, an infinity matches the same infinity, every
    other value within max(2e-3, 8e-3 * |expected|).  Applied as a hard bound on the chains of two
    roundings, where the 1-ulp bound only holds stage by stage."""
    a = orc.bf16_decode(np.asarray(got)).astype(np.float64).reshape(-1)
    e = orc.bf16_decode(np.asarray(want)).astype(np.float64).reshape(-1)
    nan_e, inf_e = np.isnan(e), np.isinf(e)
    assert np.array_equal(np.isnan(a), nan_e), f"{what}: NaN classification differs"
    assert np.array_equal(a[inf_e], e[inf_e]), f"{what}: infinity classification differs"
    fin = ~(nan_e | inf_e)
    tol = np.maximum(2.0e-3, np.abs(e[fin]) * 8.0e-3)
    err = np.abs(a[fin] - e[fin])
    bad = np.nonzero(err > tol)[0]
    assert bad.size == 0, (f"{what}: {bad.size} elements beyond max(2e-3, 8e-3|e|); worst {err[bad].max():.3e} "
                           f"at expected {e[fin][bad[np.argmax(err[bad])]]:.6g}")


def assert_bits_equal(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    bad = np.nonzero(got.reshape(-1) != want.reshape(-1))[0]
    assert bad.size == 0, f"{what}: {bad.size} mismatching elements, first at {bad[:5]}"
