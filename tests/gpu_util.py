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


def scratch_for(rows, rows_per_scale, fill=0x7FFFFFFF):
    """The caller-owned scratch of the NVFP4 entry points, pre-filled with garbage: stale contents
    must not matter."""
    words = capi.lib().q3x_b200_nvfp4_scratch_words(rows, rows_per_scale)
    return empty_like_dev((words,), dtype=np.uint32, fill=fill)


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


def assert_bits_equal(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    bad = np.nonzero(got.reshape(-1) != want.reshape(-1))[0]
    assert bad.size == 0, f"{what}: {bad.size} mismatching elements, first at {bad[:5]}"
