"""The entry point for callers that cannot allocate device memory
(q3x_b200_residual_add_rms_norm_nvfp4_static_scratch): its scratch words live in a fixed device
array inside the library instead of coming from the caller.  Such callers are, for example, code
running in a stream callback, and plugins that only ever receive their input and output tensors.

The test calls it through the C ABI twice in a row on different inputs (the array keeps the first
call's contents, so the second call shows that stale words do no harm) and requires every output to
be bit-identical to the regular entry point, which takes caller-owned scratch.  It also checks that
a call beyond the array's capacity is refused before anything runs.  The file is named so that
pytest collects it last.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests import fixtures as fx

pytestmark = pytest.mark.gpu
EPS = 1e-6


@pytest.fixture(scope="module")
def g():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_util

    orc.build()
    gpu_util.capi.load()
    return gpu_util


def run_both(g, tokens, rps, seed):
    hidden = 5120
    rng = np.random.default_rng([tokens, rps, seed])
    left, right = fx.normal_bf16(rng, (tokens, hidden), 1.0 + seed), fx.normal_bf16(rng, (tokens, hidden))
    w = fx.normal_bf16(rng, (hidden,), 0.02)
    groups = 1 if rps == 0 else (tokens + rps - 1) // rps
    dl, dr, dw = g.Dev(left), g.Dev(right), g.Dev(w)

    def outputs():
        return dict(res=g.empty_like_dev((tokens, hidden)), nrm=g.empty_like_dev((tokens, hidden)),
                    gs=g.empty_like_dev((groups,), dtype=np.float32),
                    codes=g.empty_like_dev((tokens, hidden // 2), dtype=np.uint8),
                    scales=g.empty_like_dev((tokens, hidden // 16), dtype=np.uint8))

    a, b = outputs(), outputs()
    scratch = g.scratch_for(tokens, rps)
    g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4", dl, dr, dw, tokens, hidden, EPS, rps, a["res"], a["nrm"],
                 scratch, a["gs"], a["codes"], a["scales"], None)
    g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4_static_scratch", dl, dr, dw, tokens, hidden, EPS, rps,
                 b["res"], b["nrm"], b["gs"], b["codes"], b["scales"], None)
    g.sync()
    for key in a:
        got, want = b[key].get(), a[key].get()
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"{key} differs from the regular entry point"
        assert b[key].guards_intact()
    # and the regular entry point is itself right: codes follow from its normalised rows
    want_c, want_s, want_g = orc.nvfp4_quantize(a["nrm"].get(), rps)
    assert np.array_equal(b["codes"].get(), want_c) and np.array_equal(b["scales"].get(), want_s)
    assert np.array_equal(b["gs"].get().view(np.uint32), want_g.view(np.uint32))


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row(g):
    run_both(g, 700, 512, seed=0)   # two scale groups
    run_both(g, 300, 0, seed=1)     # fewer rows, one group: the array still holds the first call's words
    run_both(g, 700, 512, seed=2)


def test_static_scratch_entry_refuses_what_does_not_fit(g):
    limit = g.capi.lib().q3x_b200_static_scratch_max_tokens()
    assert limit == 16384
    fake = 0x10000  # never dereferenced: the call must fail on the host
    st = g.capi.call("q3x_b200_residual_add_rms_norm_nvfp4_static_scratch", fake, fake + (1 << 30), fake + (2 << 30),
                     limit + 1, 5120, EPS, 512, fake + (3 << 30), fake + (4 << 30), fake + (5 << 30), fake + (6 << 30),
                     fake + (7 << 30), None)
    assert st == g.capi.CUDA_ERROR_INVALID_VALUE
    # one row per scale group needs two words per row: more than the array holds at this size
    st = g.capi.call("q3x_b200_residual_add_rms_norm_nvfp4_static_scratch", fake, fake + (1 << 30), fake + (2 << 30),
                     limit, 5120, EPS, 1, fake + (3 << 30), fake + (4 << 30), fake + (5 << 30), fake + (6 << 30),
                     fake + (7 << 30), None)
    assert st == g.capi.CUDA_ERROR_INVALID_VALUE
