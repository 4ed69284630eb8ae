"""W4A8 on the GPU against the CPU oracle (the restatement of the reference's gemm_ref), bit for bit: Q4_K and Q6_K,
bf16 stores and fp32 residual adds, several row counts and live counts (padded buckets), a fused mixed-kind projection
(tests/test_w4a8.py:45-75).  Activations: N(0, 1) with k / 64 outlier channels x20 (tests/test_w4a8.py:26-30)."""
import numpy as np
import pytest
import torch

import oracle
from prism_b200 import quant, synth, w4a8
from util import bf16_from_bits, first_diff, n_rows, np_bits, same

pytestmark = pytest.mark.gpu


def weights(kind, n, k, seed):
    w = synth.weights(n, k, seed)
    return w4a8.repack(synth.q4_k(w) if kind == "q4k" else synth.q6_k(w)), w


def ref_gemm(xq, a, xs, w, epi, live, out=None):
    g = lambda t: None if t is None else t.numpy()          # noqa: E731
    return oracle.w4a8_gemm(xq, a, xs, w.kind, g(w.q), g(w.sc), g(w.mn), g(w.d), g(w.dm), epi=epi, live=live, out=out)


@pytest.mark.parametrize("kind", ["q4k", "q6k"])
@pytest.mark.parametrize("m,live,n,k", [(1, 1, 256, 512), (7, 7, 320, 2560), (64, 50, 1024, 5120), (300, 300, 192, 1024),
                                        (130, 127, 4100, 512), (17, 17, 1000, 1024), (48, 33, 132, 768),
                                        (16, 16, 5120, 5120), (2, 2, 1000, 1024), (4, 3, 4100, 2560), (3, 3, 132, 768),
                                        (4, 4, 100, 512), (1, 1, 5120, 5120), (8, 8, 1000, 1024), (6, 5, 320, 2560),
                                        (8, 8, 5120, 5120), (5, 5, 132, 768)])
def test_gemm_bits(dev, kind, m, live, n, k):
    w, wf = weights(kind, n, k, seed=n + k)
    x = synth.activations(m, k, seed=m, outliers=k // 64)
    xq, a, xs = oracle.quant_g(np_bits(x))
    ref0 = ref_gemm(xq, a, xs, w, 0, live)
    base = torch.randn(m, n, generator=torch.Generator().manual_seed(4))
    ref1 = ref_gemm(xq, a, xs, w, 1, live, out=base.numpy())
    wd = w.to(dev)
    nr = n_rows(live, dev)
    xqd, ad, xsd = (torch.from_numpy(t).to(dev) for t in (xq, a, xs))
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
    w4a8.gemm(xqd, ad, xsd, wd, out, nr, epi=0)
    assert same(out, bf16_from_bits(ref0)), first_diff(np_bits(out), ref0)
    res = base.to(dev)
    w4a8.gemm(xqd, ad, xsd, wd, res, nr, epi=1)
    assert same(res, ref1), first_diff(res.cpu().numpy(), ref1)
    if m <= 16:
        # K splits of the few-rows kernel leave the chain's terms in a workspace and one CTA adds them in order: the
        # same bits for every split
        for cfg in (1, 2, 5):
            out = torch.zeros(m, n, dtype=torch.bfloat16, device=dev)
            w4a8.gemm(xqd, ad, xsd, wd, out, nr, epi=0, cfg=cfg)
            assert same(out, bf16_from_bits(ref0)), (cfg, first_diff(np_bits(out), ref0))
            res = base.to(dev)
            w4a8.gemm(xqd, ad, xsd, wd, res, nr, epi=1, cfg=cfg)
            assert same(res, ref1), (cfg, first_diff(res.cpu().numpy(), ref1))
    # the quantized product stays close to the unquantized one (tests/test_w4a8.py:73-75: a few per cent)
    kq = synth.q4_k(wf) if kind == "q4k" else synth.q6_k(wf)
    true = x[:live].float() @ kq.dequant().T
    got = oracle.bf16_to_f32(ref0)[:live]
    assert np.linalg.norm(got - true.numpy()) / np.linalg.norm(true.numpy()) < 0.05


def test_fused_mixed_projection(dev):
    """q | k as Q4_K and v as Q6_K in one output buffer (the Q4_K_M convention), through rows_g on the GPU."""
    k, m = 1024, 20
    wq = synth.weights(384, k, 1)
    wv = synth.weights(128, k, 2)
    kqs = [synth.q4_k(wq[:256]), synth.q4_k(wq[256:]), synth.q6_k(wv)]
    segs = w4a8.segments(kqs, dev)
    assert [(s[0].kind, s[0].n, s[1]) for s in segs] == [("q4k", 384, 0), ("q6k", 128, 384)]
    assert w4a8.seg_width(segs) == 512
    x = synth.activations(m, k, seed=9, outliers=16)
    nr = n_rows(m, dev)
    q = torch.empty(m, k, dtype=torch.int8, device=dev)
    a = torch.empty(k // 256, m, device=dev)
    xs = torch.empty(k // 256, m, 16, dtype=torch.int8, device=dev)
    quant.rows_g(x.to(dev), q, a, xs, nr, m)
    out = torch.zeros(m, 512, dtype=torch.bfloat16, device=dev)
    w4a8.gemm_segs(q, a, xs, segs, out, nr)
    rq, ra, rxs = oracle.quant_g(np_bits(x))
    for (w, off) in segs:
        ref = ref_gemm(rq, ra, rxs, w.to("cpu"), 0, m)
        assert same(out[:, off:off + w.n].contiguous(), bf16_from_bits(ref)), w.kind
    sub = w4a8.seg_rows(segs, 300, 450)
    assert [(s[0].kind, s[0].n, s[1]) for s in sub] == [("q4k", 84, 0), ("q6k", 66, 84)]
