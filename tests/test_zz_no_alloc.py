"""The allocation-free split-K GEMM entry point (pb_w8a8_gemm_static) against the ordinary one, through the C ABI.

Callers that cannot allocate device memory - a plugin inside another runtime's memory pool, a launch-only replay
thread, code that runs during stream capture - use the variant whose split-K scratch is a fixed array in the library's
device image.  It must give the ordinary entry point's bits, on two calls in a row (the array keeps the first call's
partial sums and counters), refuse products whose scratch does not fit, and allocate nothing.  This file sorts last so
that a run that stops at the first failure has already run every other test."""
import pytest
import torch

from prism_b200 import _lib, w8a8
from util import n_rows, rand_w8a8

pytestmark = pytest.mark.gpu


def call_static(L, a, sa, w, sw, out, nr, epi, split):
    M, K = a.shape
    return L.pb_w8a8_gemm_static(a.data_ptr(), sa.data_ptr(), w.data_ptr(), sw.data_ptr(), out.data_ptr(),
                                 out.stride(0), nr.data_ptr(), M, w.shape[0], K, epi, split,
                                 torch.cuda.current_stream().cuda_stream)


def call_plain(L, a, sa, w, sw, out, nr, epi, split, ws, counters):
    M, K = a.shape
    return L.pb_w8a8_gemm(a.data_ptr(), sa.data_ptr(), w.data_ptr(), sw.data_ptr(), out.data_ptr(), out.stride(0),
                          nr.data_ptr(), M, w.shape[0], K, K, epi, split, 0, ws.data_ptr(), ws.numel(),
                          counters.data_ptr(), counters.numel(), 0, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,N,K,live,split", [(16, 5120, 5120, 16, 4), (64, 1000, 2560, 50, 5), (8, 7168, 5120, 8, 5)])
def test_static_scratch_matches_workspace_entry_point(dev, lib, M, N, K, live, split):
    a, w, sa, sw = (t.to(dev) for t in rand_w8a8(M, N, K, seed=M + N))
    sa, sw = sa.view(-1), sw.view(-1)
    nr = n_rows(live, dev)
    ws = torch.empty(lib.pb_w8a8_workspace_bytes(M, N, split), dtype=torch.uint8, device=dev)
    counters = torch.zeros(lib.pb_w8a8_counters(M, N), dtype=torch.int32, device=dev)
    want0 = torch.full((M, N), 3.0, dtype=torch.bfloat16, device=dev)
    assert call_plain(lib, a, sa, w, sw, want0, nr, 0, split, ws, counters) == 0
    base = torch.randn(M, N, device=dev)
    want1 = base.clone()
    assert call_plain(lib, a, sa, w, sw, want1, nr, 1, split, ws, counters) == 0
    # a warm-up call first: the library looks up the array's address on its first call on a device, and the CUDA
    # runtime may load the kernel's module lazily - neither belongs to the steady state measured below
    warm = torch.full((M, N), 3.0, dtype=torch.bfloat16, device=dev)
    assert call_static(lib, a, sa, w, sw, warm, nr, 0, split) == 0
    torch.cuda.synchronize()
    for _ in range(2):                                   # twice in a row: the array keeps the previous call's contents
        got0 = torch.full((M, N), 3.0, dtype=torch.bfloat16, device=dev)
        got1 = base.clone()
        torch.cuda.synchronize()
        # the device's free bytes, as the driver counts them: a cudaMalloc made anywhere in this process - torch's
        # allocator or the library itself - would lower the figure (torch's own counters see only torch's)
        free_before = torch.cuda.mem_get_info(dev)[0]
        mark = torch.cuda.memory_allocated(dev)
        assert call_static(lib, a, sa, w, sw, got0, nr, 0, split) == 0
        assert call_static(lib, a, sa, w, sw, got1, nr, 1, split) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] >= free_before    # no device allocation by anyone during the calls
        assert torch.cuda.memory_allocated(dev) == mark          # and nothing through torch's allocator
        assert torch.equal(got0.view(torch.int16), want0.view(torch.int16))
        assert torch.equal(got1.view(torch.int32), want1.view(torch.int32))
        assert bool((got0[live:] == 3).all())


def test_static_scratch_limits(dev, lib):
    """A product whose partial sums do not fit the 16 MiB array is refused with PB_TOO_LARGE; many rows are
    unsupported; one split needs no scratch at all."""
    assert lib.pb_w8a8_static_scratch_bytes() == 16 << 20
    M, N, K = 64, 34816, 5120
    a, w, sa, sw = (t.to(dev) for t in rand_w8a8(M, N, K, seed=1))
    nr = n_rows(M, dev)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    assert lib.pb_w8a8_workspace_bytes(M, N, 8) > (16 << 20)
    assert call_static(lib, a, sa.view(-1), w, sw.view(-1), out, nr, 0, 8) == 5
    assert not bool(out.any())
    assert call_static(lib, a, sa.view(-1), w, sw.view(-1), out, nr, 0, 1) == 0
    ref = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(a, sa.view(-1), w, sw.view(-1), ref, nr, K, cfg=1)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    big = torch.zeros(65, K, dtype=torch.int8, device=dev)
    assert lib.pb_w8a8_gemm_static(big.data_ptr(), sa.data_ptr(), w.data_ptr(), sw.data_ptr(), out.data_ptr(), N,
                                   nr.data_ptr(), 65, N, K, 0, 2, None) == 2
