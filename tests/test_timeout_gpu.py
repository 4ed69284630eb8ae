"""A bounded device-side wait that runs out: the kernel must record PB_DEVICE_TIMEOUT, leave through its abort path
(every role out of its loop, tensor memory freed) and return, and the next launch on the same context must be correct.

The failure is injected on the host (pb_test_drop_loads): the many-rows W8A8 kernel's producer requests no tiles, so the
barrier its MMA thread waits for is one that nothing completes.  The bound is lowered to 2 ms for the test
(pb_set_wait_limit_ns) and restored afterwards.  Nothing here faults, traps or spins without a bound."""
import pytest
import torch

import oracle
from prism_b200 import _lib, w8a8
from util import bf16_from_bits, n_rows, rand_w8a8, same

pytestmark = pytest.mark.gpu


def test_wait_expires_status_4_then_clean_launch(dev, lib):
    M, N, K = 256, 512, 1024
    a, w, sa, sw = rand_w8a8(M, N, K, seed=11)
    ad, wd, sad, swd = a.to(dev), w.to(dev), sa.to(dev).view(-1), sw.to(dev).view(-1)
    nr = n_rows(M, dev)
    want = bf16_from_bits(oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), K, 0, M))
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(ad, sad, wd, swd, out, nr, K)                          # the healthy kernel first
    torch.cuda.synchronize()
    assert same(out, want)
    assert _lib.device_status(reset=True)[0] == 0
    assert lib.pb_set_wait_limit_ns(2_000_000) == 0
    assert lib.pb_test_drop_loads(1) == 0
    try:
        junk = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        w8a8.gemm(ad, sad, wd, swd, junk, nr, K)                     # its consumers wait for tiles nobody requested
        torch.cuda.synchronize()                                     # returns: the waits were bounded
        code, where = _lib.device_status(reset=True)
    finally:
        lib.pb_test_drop_loads(0)
        lib.pb_set_wait_limit_ns(0)
    assert code == 4, code
    assert where & 0xF00 in (0x300, 0x400), hex(where)               # the MMA thread's or an epilogue warp's wait
    assert _lib.device_status(reset=False)[0] == 0                   # the word was cleared
    # the context is intact and tensor memory was given back: the same product again, and a split-K one
    out2 = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(ad, sad, wd, swd, out2, nr, K)
    out3 = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(ad, sad, wd, swd, out3, nr, K, cfg=2)
    torch.cuda.synchronize()
    assert same(out2, want) and same(out3, want)
