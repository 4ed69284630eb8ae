"""The vocabulary head on Q8_0 weights (kernels/decode.py:113-160, :351-364): final norm + int8 per 32 inputs, then the
per-32-group GEMM with a plain fp32 store, against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from prism_b200 import decode, synth
from util import first_diff, n_rows, rand_w8a8, same

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,HID,live", [(1, 5120, 1), (9, 5120, 7), (64, 2048, 64)])
def test_head_quant(dev, B, HID, live):
    g = torch.Generator().manual_seed(B + HID)
    h = torch.randn(B, HID, generator=g) * 3
    w = torch.rand(HID, generator=g) + 0.5
    rq, rs = oracle.head_quant(h.numpy(), w.numpy(), 1e-6, live)
    q = torch.zeros(B, HID, dtype=torch.int8, device=dev)
    s = torch.zeros(B, HID // 32, device=dev)
    decode.head_quant(h.to(dev), w.to(dev), q, s, n_rows(live, dev), B, 1e-6)
    assert np.abs(q.cpu().numpy().astype(int) - rq.astype(int)).max() <= 1
    assert (q.cpu().numpy() != rq).mean() < 0.01
    assert np.allclose(s.cpu().numpy()[:live], rs[:live], rtol=1e-5)
    assert not bool(q[live:].any())


@pytest.mark.parametrize("B,N,K,live", [(1, 4000, 1024, 1), (16, 24832, 5120, 13), (64, 1000, 2560, 64)])
def test_head_q8(dev, B, N, K, live):
    """logits = the groups' sums in order, acc = fma(float(a_g . w_g) * a_s[g], w_s[g], acc) - what the reference's
    kernel computes once its compiler has fused `acc += (ai * sa) * sw` (pinned by the recorded reference output,
    tests/test_reference_kernels.py::test_head) - with the scales as the file keeps them (fp16, group-major): the
    oracle's bits; rows >= live untouched."""
    a, w, sa, sw = rand_w8a8(B, N, K, seed=N, groups=K // 32)
    sw16 = sw.to(torch.float16)                                     # the file's precision
    ref = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw16.float().numpy(), 32, 4, live)
    ws_file = sw16.t().contiguous()                                 # [K / 32, N]
    out = torch.full((B, N), 7.0, device=dev)
    decode.head_q8(a.to(dev), sa.to(dev), w.to(dev), ws_file.to(dev), out, n_rows(live, dev), B)
    got = out.cpu().numpy()
    assert np.array_equal(got[:live], ref[:live]), first_diff(got[:live], ref[:live])
    assert bool((out[live:] == 7.0).all())
