"""Launch-contract tests on the GPU: asynchronous launches on a caller-supplied non-default stream,
a stale CUDA error left by unrelated work is cleared (the reference's launch_after_stale pattern,
tests/decode_ops_cuda_test.cu:374-387), rejected calls leave the outputs untouched, and the
operators can be captured into a CUDA graph and replayed."""
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


def test_device_is_blackwell(g):
    major, minor = torch.cuda.get_device_capability(0)
    assert (major, minor) == (10, 0), "the library is built for sm_100a only"


def test_stale_error_is_cleared_and_stream_is_honoured(g):
    rng = np.random.default_rng(41)
    a, b = fx.normal_bf16(rng, (4096,)), fx.normal_bf16(rng, (4096,))
    da, db = g.Dev(a), g.Dev(b)
    out = g.empty_like_dev((4096,))
    stream = torch.cuda.Stream()
    L = g.capi.lib()
    assert L.q3x_b200_debug_stale_error(1) != 0          # a stale error is now pending
    with torch.cuda.stream(stream):
        st = g.capi.call("q3x_b200_residual_add", da, db, 4096, out, stream.cuda_stream)
    assert st == 0, "the launch reports its own status, not the stale error"
    assert L.q3x_b200_debug_stale_error(0) == 0
    stream.synchronize()
    g.assert_bits_equal(out.get(), orc.residual_add(a, b), "residual add on a side stream")


def test_rejected_call_writes_nothing(g):
    rng = np.random.default_rng(42)
    x = fx.normal_bf16(rng, (4, 5120))
    w = fx.normal_bf16(rng, (5120,), 0.02)
    dx, dw = g.Dev(x), g.Dev(w)
    out = g.empty_like_dev((4, 5120), fill=0x7777)
    assert g.capi.call("q3x_b200_rms_norm", dx, dw, 4, 5120, 0.0, 1, out, None) == g.capi.CUDA_ERROR_INVALID_VALUE
    # partial overlap of output and input
    assert g.capi.call("q3x_b200_rms_norm", dx, dw, 2, 5120, EPS, 1, dx.ptr_at(16), None) == g.capi.CUDA_ERROR_INVALID_VALUE
    g.sync()
    assert np.all(out.get() == 0x7777) and np.array_equal(dx.get(), x)
    # misaligned pointers on a kernel that only has a 128-bit path
    C_ = 10240
    raw = g.Dev(fx.normal_bf16(rng, (2, C_)), misalign=1)
    st = g.capi.call("q3x_b200_causal_conv1d_silu", raw, 2, C_, g.Dev(np.zeros((C_, 4), np.uint16)),
                     g.Dev(np.zeros((C_, 3), np.uint16)), g.empty_like_dev((2, C_)), None)
    assert st == g.capi.CUDA_ERROR_NOT_SUPPORTED


def test_graph_capture_and_replay(g):
    rng = np.random.default_rng(43)
    tokens, hidden = 64, 5120
    left, right = fx.normal_bf16(rng, (tokens, hidden)), fx.normal_bf16(rng, (tokens, hidden))
    w = fx.normal_bf16(rng, (hidden,), 0.02)
    dl, dr, dw = g.Dev(left), g.Dev(right), g.Dev(w)
    res, nrm = g.empty_like_dev((tokens, hidden)), g.empty_like_dev((tokens, hidden))
    amax = g.scratch_for(tokens, 0)
    gs = g.empty_like_dev((1,), dtype=np.float32)
    codes = g.empty_like_dev((tokens, hidden // 2), dtype=np.uint8)
    scales = g.empty_like_dev((tokens, hidden // 16), dtype=np.uint8)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            s = torch.cuda.current_stream().cuda_stream
            g.capi.check("q3x_b200_residual_add_rms_norm_nvfp4", dl, dr, dw, tokens, hidden, EPS, 0, res, nrm, amax,
                         gs, codes, scales, s)
    for _ in range(3):
        graph.replay()
    g.sync()
    want_r, want_n = orc.residual_add_rms_norm(left, right, w, EPS)
    g.assert_bits_equal(res.get(), want_r, "residual from a replayed graph")
    want_c, want_s, want_g = orc.nvfp4_quantize(nrm.get(), 0)
    g.assert_bits_equal(codes.get(), want_c, "codes from a replayed graph")
    g.assert_bits_equal(scales.get(), want_s, "scales from a replayed graph")


def test_full_size_properties(g):
    """Size-independent properties at the configured sizes (8192-token GDN panel, 17408-wide MLP):
    chunk-splitting invariance of the conv, idempotent re-quantisation of dequantised codes, and the
    merged / split SwiGLU layouts agreeing bit for bit."""
    gen = torch.Generator(device="cuda").manual_seed(7)
    T, C_ = 8192, 10240
    raw = torch.randn(T, C_, generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(C_, 4, generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
    out_a, out_b = torch.empty_like(raw), torch.empty_like(raw)
    h_a = torch.zeros(C_, 3, device="cuda", dtype=torch.bfloat16)
    h_b = torch.zeros_like(h_a)
    g.capi.check("q3x_b200_causal_conv1d_silu", raw, T, C_, w, h_a, out_a, None)
    cut = 4099
    g.capi.check("q3x_b200_causal_conv1d_silu", raw, cut, C_, w, h_b, out_b, None)
    g.capi.check("q3x_b200_causal_conv1d_silu", raw.data_ptr() + cut * C_ * 2, T - cut, C_, w, h_b,
                 out_b.data_ptr() + cut * C_ * 2, None)
    g.sync()
    assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
    assert torch.equal(h_a.view(torch.int16), h_b.view(torch.int16))
    assert torch.equal(h_a.view(torch.int16), raw[-3:].t().contiguous().view(torch.int16))
    # torch fp32 reference of the same op, compared in bf16 ulps on a slice
    x = torch.cat([torch.zeros(3, C_, device="cuda"), raw.float()])
    acc = sum(x[j:j + T] * w[:, j].float() for j in range(4))
    ref = (acc * torch.sigmoid(acc)).to(torch.bfloat16)
    diff = (out_a.float() - ref.float()).abs()
    assert (diff <= ref.float().abs() * 2 ** -7 + 1e-30).all()

    I = 17408
    merged = torch.randn(2048, 2 * I, generator=gen, device="cuda").to(torch.bfloat16)
    o1 = torch.empty(2048, I, device="cuda", dtype=torch.bfloat16)
    o2 = torch.empty_like(o1)
    gate, up = merged[:, :I].contiguous(), merged[:, I:].contiguous()
    g.capi.check("q3x_b200_silu_mul_merged", merged, 2048, I, o1, None)
    g.capi.check("q3x_b200_silu_mul", gate, up, 2048 * I, o2, None)
    g.sync()
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
    ref = (torch.nn.functional.silu(gate.float()) * up.float()).to(torch.bfloat16)
    assert ((o1.float() - ref.float()).abs() <= ref.float().abs() * 2 ** -7 + 1e-30).all()

    # NVFP4 at full width: the reconstruction error is bounded by the block scale, and the largest
    # element of every scale group lands on +-6 under the largest scale (448)
    x = o1[:1024]
    amax = torch.zeros(g.capi.lib().q3x_b200_nvfp4_scratch_words(1024, 512), device="cuda", dtype=torch.int32)
    gs = torch.empty(2, device="cuda", dtype=torch.float32)
    codes = torch.empty(1024, I // 2, device="cuda", dtype=torch.uint8)
    scales = torch.empty(1024, I // 16, device="cuda", dtype=torch.uint8)
    g.capi.check("q3x_b200_nvfp4_quantize_dynamic", x, 1024, I, 512, amax, gs, codes, scales, None)
    g.sync()
    e2 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], device="cuda")
    nib = torch.stack([codes & 0xF, codes >> 4], dim=-1).reshape(1024, I).long()
    d = scales.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=1) * gs.repeat_interleave(512)[:, None]
    deq = e2[nib] * d
    assert ((deq - x.float()).abs() <= 1.4 * d + 1e-30).all()
    for grp in range(2):
        xs = x[grp * 512:(grp + 1) * 512].float().abs()
        top = xs.max()
        assert gs[grp].item() == (top / 2688.0).item()
        where = (xs == top).nonzero()[0]
        r, c = int(where[0]) + grp * 512, int(where[1])
        assert scales[r, c // 16].item() == 0x7E and (nib[r, c].item() & 7) == 7
