"""Activation quantizers and the fold on the GPU against the CPU oracle: bit for bit where the kernel does no
transcendental arithmetic (rows_q8, quant_rows, rows_g, fold), within one int8 step for SwiGLU (exp differs in its
last bits between a GPU and libm; tests/test_w4a8.py:91-102 sets the same bar for the reference's fused producers)."""
import numpy as np
import pytest
import torch

import oracle
from prism_b200 import quant, synth, w8a8
from util import first_diff, n_rows, np_bits, same

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,K,live", [(1, 5120, 1), (33, 5120, 30), (16, 17408, 16), (7, 2560, 7), (5, 1000, 5),
                                      (3, 40000, 3), (9, 264, 9)])
@pytest.mark.parametrize("smooth", [False, True])
def test_rows_q8(dev, T, K, live, smooth):
    x = synth.activations(T, K, seed=T + K)
    inv = torch.exp(torch.randn(K, generator=torch.Generator().manual_seed(K)) * 0.1) if smooth else None
    rq, rs = oracle.quant_rows(np_bits(x), inv_s=None if inv is None else inv.numpy(), live=live)
    q = torch.full((T, K), 99, dtype=torch.int8, device=dev)
    s = torch.full((T,), -1.0, device=dev)
    quant.rows_q8(x.to(dev), None if inv is None else inv.to(dev), q, s, n_rows(live, dev), T)
    assert same(q[:live], rq[:live]), first_diff(q[:live].cpu().numpy(), rq[:live])
    assert same(s[:live], rs[:live, 0])
    assert bool((q[live:] == 99).all()) and bool((s[live:] == -1).all())
    # fp32 input
    xf = x.float() * 1.001
    rq, rs = oracle.quant_rows(xf.numpy(), inv_s=None if inv is None else inv.numpy(), live=live)
    quant.rows_q8(xf.to(dev), None if inv is None else inv.to(dev), q, s, n_rows(live, dev), T)
    assert same(q[:live], rq[:live]) and same(s[:live], rs[:live, 0])


def test_rows_q8_tp_modes(dev):
    """Modes 1 / 2 (kernels/quant.py:301-304): column halves quantized with the whole row's maximum give the whole
    row's int8 values and scale."""
    T, K = 9, 5120
    x = synth.activations(T, K, seed=3)
    rq, rs = oracle.quant_rows(np_bits(x))
    nr = n_rows(T, dev)
    halves = [x[:, :K // 2].contiguous().to(dev), x[:, K // 2:].contiguous().to(dev)]
    amax = [torch.zeros(T, device=dev) for _ in halves]
    qs = [torch.empty(T, K // 2, dtype=torch.int8, device=dev) for _ in halves]
    ss = [torch.empty(T, device=dev) for _ in halves]
    for h, am, q, s in zip(halves, amax, qs, ss):
        quant.rows_q8(h, None, q, s, nr, T, mode=1, amax=am)
    tot = torch.maximum(amax[0], amax[1])
    for h, q, s in zip(halves, qs, ss):
        quant.rows_q8(h, None, q, s, nr, T, mode=2, amax=tot.clone())
    assert same(torch.cat(qs, 1), rq) and same(ss[0], rs[:, 0]) and same(ss[1], rs[:, 0])


@pytest.mark.parametrize("T,K,gk", [(4, 5120, 32), (3, 1024, 128), (17, 512, 256), (2, 17408, 32)])
def test_quant_rows_groups(dev, T, K, gk):
    x = synth.activations(T, K, seed=gk)
    rq, rs = oracle.quant_rows(np_bits(x), gk)
    q, s = w8a8.quant_rows(x.to(dev), gk)
    assert same(q, rq) and same(s, rs)


@pytest.mark.parametrize("T,K,live", [(33, 2560, 33), (5, 5120, 4), (2, 17408, 2)])
def test_rows_g(dev, T, K, live):
    """rows_g against the oracle's quantize_ref restatement (tests/test_w4a8.py:80-90)."""
    x = synth.activations(T, K, seed=K, outliers=K // 64)
    rq, ra, rxs = oracle.quant_g(np_bits(x), live)
    q = torch.zeros(T, K, dtype=torch.int8, device=dev)
    a = torch.zeros(K // 256, T, device=dev)
    xs = torch.zeros(K // 256, T, 16, dtype=torch.int8, device=dev)
    quant.rows_g(x.to(dev), q, a, xs, n_rows(live, dev), T)
    assert same(q, rq) and same(a, ra) and same(xs, rxs)


@pytest.mark.parametrize("T,FF,live", [(5, 17408, 5), (3, 1024, 2), (2, 4352, 2)])
def test_swiglu_q8(dev, T, FF, live):
    g = torch.Generator().manual_seed(FF)
    gu = (torch.randn(T, 2 * FF, generator=g) * 2).to(torch.bfloat16)
    rq, rs = oracle.swiglu_q8(np_bits(gu), live=live)
    q = torch.zeros(T, FF, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    quant.swiglu_q8(gu.to(dev), None, q, s, n_rows(live, dev), T)
    assert np.abs(q.cpu().numpy().astype(int) - rq.astype(int)).max() <= 1
    assert np.allclose(s.cpu().numpy()[:live], rs[:live], rtol=1e-5)
    assert not bool(q[live:].any())


def test_fold_odd(dev):
    """fold with N not a multiple of 4 and a strided residual."""
    T, N, S = 5, 30, 3
    g = torch.Generator().manual_seed(0)
    slots = torch.randint(-10 ** 6, 10 ** 6, (S, T, N), generator=g, dtype=torch.int32)
    sa, sw = torch.rand(T, generator=g) * 1e-2, torch.rand(N, generator=g) * 1e-3
    h = torch.randn(T, N, generator=g)
    ref = oracle.fold(h.numpy(), slots.numpy(), sa.numpy(), sw.numpy(), live=4)
    hd = h.to(dev)
    quant.fold(hd, slots.to(dev), w8a8.Deferred(S, sa.to(dev), sw.to(dev)), n_rows(4, dev), T)
    assert same(hd, ref)


@pytest.mark.parametrize("T,K,live", [(300, 5120, 290), (1000, 2560, 1000), (260, 17408, 257), (512, 264, 512)])
def test_rows_q8_many_rows(dev, T, K, live):
    """From 256 rows the row-pipelined kernel runs (persistent CTAs, rows staged in shared memory): the same bits as
    the oracle, for bf16, fp32, smoothed and strided inputs; rows >= live untouched."""
    x = synth.activations(T, K, seed=T)
    inv = torch.exp(torch.randn(K, generator=torch.Generator().manual_seed(1)) * 0.1)
    nr = n_rows(live, dev)
    for xin, iv in ((x, None), (x, inv), (x.float() * 0.731, None)):
        ref_in = np_bits(xin) if xin.dtype == torch.bfloat16 else xin.numpy()
        rq, rs = oracle.quant_rows(ref_in, inv_s=None if iv is None else iv.numpy(), live=live)
        q = torch.full((T, K), 99, dtype=torch.int8, device=dev)
        s = torch.full((T,), -1.0, device=dev)
        quant.rows_q8(xin.to(dev), None if iv is None else iv.to(dev), q, s, nr, T)
        assert same(q[:live], rq[:live]), first_diff(q[:live].cpu().numpy(), rq[:live])
        assert same(s[:live], rs[:live, 0])
        assert bool((q[live:] == 99).all()) and bool((s[live:] == -1).all())
    wide = torch.zeros(T, K + 64, dtype=torch.bfloat16)
    wide[:, 32:32 + K] = x
    rq, rs = oracle.quant_rows(np_bits(x), live=live)
    q = torch.zeros(T, K, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    quant.rows_q8(wide.to(dev)[:, 32:32 + K], None, q, s, nr, T)
    assert same(q[:live], rq[:live]) and same(s[:live], rs[:live, 0])
    # tensor-parallel modes on the pipelined kernel
    amax = torch.zeros(T, device=dev)
    quant.rows_q8(x.to(dev), None, q, s, nr, T, mode=1, amax=amax)
    big = amax * 2
    quant.rows_q8(x.to(dev), None, q, s, nr, T, mode=2, amax=big)
    assert np.allclose(s[:live].cpu().numpy(), 2 * rs[:live, 0], rtol=1e-6)


@pytest.mark.parametrize("T,FF", [(300, 17408), (256, 1024)])
def test_swiglu_q8_many_rows(dev, T, FF):
    """The pipelined SwiGLU quantizer against the oracle within one int8 step, and bit-identical to the per-row
    kernel (the first 200 rows quantized alone)."""
    g = torch.Generator().manual_seed(FF + 1)
    gu = (torch.randn(T, 2 * FF, generator=g) * 2).to(torch.bfloat16)
    rq, rs = oracle.swiglu_q8(np_bits(gu))
    q = torch.zeros(T, FF, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    quant.swiglu_q8(gu.to(dev), None, q, s, n_rows(T, dev), T)
    assert np.abs(q.cpu().numpy().astype(int) - rq.astype(int)).max() <= 1
    assert np.allclose(s.cpu().numpy(), rs, rtol=1e-5)
    q2 = torch.zeros(200, FF, dtype=torch.int8, device=dev)
    s2 = torch.zeros(200, device=dev)
    quant.swiglu_q8(gu[:200].contiguous().to(dev), None, q2, s2, n_rows(200, dev), 200)
    assert same(q2, q[:200].contiguous()) and same(s2, s[:200].contiguous())


@pytest.mark.parametrize("T,HID,live", [(7, 5120, 5), (64, 5120, 64), (33, 2048, 33), (3, 17408, 3)])
def test_norm_q8(dev, T, HID, live):
    """RMSNorm + per-token int8 (kernels/quant.py:145-171): within one int8 step of the oracle (the sum of squares has
    no order the reference defines), the scale to 1e-5, rows >= live untouched; the row gather picks its rows."""
    g = torch.Generator().manual_seed(HID + T)
    h = torch.randn(T, HID, generator=g) * 3
    w = torch.rand(HID, generator=g) + 0.5
    rq, rs = oracle.norm_q8(h.numpy().copy(), w.numpy(), 1e-6, live=live)
    q = torch.zeros(T, HID, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    hd = h.to(dev)
    quant.norm_q8(hd, w.to(dev), q, s, n_rows(live, dev), T, 1e-6)
    assert np.abs(q.cpu().numpy().astype(int) - rq.astype(int)).max() <= 1
    assert (q.cpu().numpy() != rq).mean() < 0.01
    assert np.allclose(s.cpu().numpy()[:live], rs[:live], rtol=1e-5)
    assert not bool(q[live:].any()) and same(hd, h)
    # gather: output row i normalizes h[rows[i]]
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
    rq2, rs2 = oracle.norm_q8(h.numpy().copy(), w.numpy(), 1e-6, rows=rows.numpy())
    q2 = torch.zeros(3, HID, dtype=torch.int8, device=dev)
    s2 = torch.zeros(3, device=dev)
    quant.norm_q8(hd, w.to(dev), q2, s2, n_rows(3, dev), 3, 1e-6, rows=rows.to(dev))
    assert np.abs(q2.cpu().numpy().astype(int) - rq2.astype(int)).max() <= 1
    assert np.allclose(s2.cpu().numpy(), rs2, rtol=1e-5)


def test_norm_q8_finishes_deferred_add(dev):
    """A split-K projection's deferred residual add is finished inside norm_q8: h gets the unsplit add's bits (the
    fold's contract), then the norm runs on it."""
    T, HID, S = 9, 2048, 3
    g = torch.Generator().manual_seed(11)
    slots = torch.randint(-10 ** 6, 10 ** 6, (S, T, HID), generator=g, dtype=torch.int32)
    sa, sw = torch.rand(T, generator=g) * 1e-2, torch.rand(HID, generator=g) * 1e-3
    h = torch.randn(T, HID, generator=g)
    w = torch.rand(HID, generator=g) + 0.5
    href = h.numpy().copy()
    rq, rs = oracle.norm_q8(href, w.numpy(), 1e-6, parts=slots.numpy(), psa=sa.numpy(), psw=sw.numpy())
    assert np.array_equal(href, oracle.fold(h.numpy().copy(), slots.numpy(), sa.numpy(), sw.numpy()))
    hd = h.to(dev)
    q = torch.zeros(T, HID, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    quant.norm_q8(hd, w.to(dev), q, s, n_rows(T, dev), T, 1e-6, parts=slots.to(dev),
                  pending=w8a8.Deferred(S, sa.to(dev), sw.to(dev)))
    assert same(hd, href)
    assert np.abs(q.cpu().numpy().astype(int) - rq.astype(int)).max() <= 1
    assert np.allclose(s.cpu().numpy(), rs, rtol=1e-5)


class _GdnCfg:
    def __init__(self, v_heads, gdn_dim, eps=1e-6):
        self.v_heads, self.gdn_dim, self.eps = v_heads, gdn_dim, eps


@pytest.mark.parametrize("T,HV,D,live", [(5, 48, 128, 4), (64, 6, 128, 64), (3, 16, 64, 3), (2, 4, 256, 2)])
def test_gated_norm_q8(dev, T, HV, D, live):
    """The gated norm + quantizer (kernels/quant.py:215-246) within one int8 step of the oracle (its exponential and
    sum order differ), scales to 1e-5, the gate read from a column window of a wider projection buffer; the
    tensor-parallel modes 1 / 2 reproduce a whole-row quantization from two head shards."""
    g = torch.Generator().manual_seed(T * 100 + HV)
    o = torch.randn(T, HV * D, generator=g) * 2
    P, z_off = HV * D + 264, 136
    proj = (torch.randn(T, P, generator=g) * 1.5).to(torch.bfloat16)
    w = torch.rand(D, generator=g) + 0.5
    inv = torch.exp(torch.randn(HV * D, generator=g) * 0.1)
    rq, rs = oracle.gated_norm_q8(o.numpy(), np_bits(proj), z_off, w.numpy(), inv.numpy(), HV, D, 1e-6, live=live)
    q = torch.zeros(T, HV * D, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    cfg = _GdnCfg(HV, D)
    quant.gated_norm_q8(o.to(dev), proj.to(dev), z_off, w.to(dev), inv.to(dev), q, s, n_rows(live, dev), T, cfg)
    assert np.abs(q.cpu().numpy().astype(int) - rq.astype(int)).max() <= 1
    assert (q.cpu().numpy() != rq).mean() < 0.02
    assert np.allclose(s.cpu().numpy()[:live], rs[:live], rtol=1e-5)
    assert not bool(q[live:].any())
    if HV % 2 == 0:
        # two shards of heads: maxima stored (mode 1), combined, used (mode 2)
        h2 = HV // 2
        c2 = _GdnCfg(h2, D)
        amax = torch.zeros(2, T, device=dev)
        parts = []
        for r in range(2):
            sl = slice(r * h2 * D, (r + 1) * h2 * D)
            qs = torch.zeros(T, h2 * D, dtype=torch.int8, device=dev)
            ss = torch.zeros(T, device=dev)
            args = (o[:, sl].contiguous().to(dev), proj.to(dev), z_off + r * h2 * D, w.to(dev), inv[sl].contiguous().to(dev))
            quant.gated_norm_q8(*args, qs, ss, n_rows(live, dev), T, c2, mode=1, amax=amax[r])
            parts.append((args, qs, ss))
        both = torch.maximum(amax[0], amax[1])
        for r, (args, qs, ss) in enumerate(parts):
            quant.gated_norm_q8(*args, qs, ss, n_rows(live, dev), T, c2, mode=2, amax=both)
            assert same(qs[:live].contiguous(), q[:live, r * h2 * D:(r + 1) * h2 * D].contiguous())
            assert same(ss[:live].contiguous(), s[:live].contiguous())


def _check_g(q, s, xs, rq, rs, live):
    """A W4A8 activation triple against the oracle's: values within one int8 step, scales to 1e-5, and the group sums
    are exactly those of the kernel's own q (split as S & 63, S >> 6)."""
    qn, sn, xn = q.cpu().numpy(), s.cpu().numpy(), xs.cpu().numpy()
    assert np.abs(qn[:live].astype(int) - rq[:live].astype(int)).max() <= 1
    assert (qn[:live] != rq[:live]).mean() < 0.02
    assert np.allclose(sn[:, :live], rs[:, :live], rtol=1e-5)
    K = qn.shape[1]
    S = qn[:live].astype(np.int32).reshape(live, K // 256, 8, 32).sum(-1)          # [live, K/256, 8]
    got = xn[:, :live].astype(np.int32)                                               # [K/256, live, 16]
    assert np.array_equal(got[..., :8], (S & 63).transpose(1, 0, 2))
    assert np.array_equal(got[..., 8:], (S >> 6).transpose(1, 0, 2))


def test_w4a8_producer_twins(dev):
    """swiglu_g, norm_g, gated_norm_g (kernels/quant.py:333-411): the fused producers through the per-256 quantizer."""
    g = torch.Generator().manual_seed(21)
    T, live = 9, 7
    nr = n_rows(live, dev)

    def outs(K):
        return (torch.zeros(T, K, dtype=torch.int8, device=dev), torch.zeros(K // 256, T, device=dev),
                torch.zeros(K // 256, T, 16, dtype=torch.int8, device=dev))
    FF = 1536
    gu = (torch.randn(T, 2 * FF, generator=g) * 2).to(torch.bfloat16)
    q, s, xs = outs(FF)
    quant.swiglu_g(gu.to(dev), q, s, xs, nr, T)
    _check_g(q, s, xs, *oracle.swiglu_g(np_bits(gu), live)[:2], live)
    HID = 5120
    h = torch.randn(T, HID, generator=g) * 3
    w = torch.rand(HID, generator=g) + 0.5
    q, s, xs = outs(HID)
    quant.norm_g(h.to(dev), w.to(dev), q, s, xs, nr, T, 1e-6)
    _check_g(q, s, xs, *oracle.norm_g(h.numpy(), w.numpy(), 1e-6, live)[:2], live)
    HV, D = 48, 128
    o = torch.randn(T, HV * D, generator=g) * 2
    P, z_off = HV * D + 264, 136
    proj = (torch.randn(T, P, generator=g) * 1.5).to(torch.bfloat16)
    wd = torch.rand(D, generator=g) + 0.5
    q, s, xs = outs(HV * D)
    quant.gated_norm_g(o.to(dev), proj.to(dev), z_off, wd.to(dev), q, s, xs, nr, T, _GdnCfg(HV, D))
    _check_g(q, s, xs, *oracle.gated_norm_g(o.numpy(), np_bits(proj), z_off, wd.numpy(), HV, D, 1e-6, live)[:2], live)
