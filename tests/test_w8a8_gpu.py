"""W8A8 GEMM on the GPU against the CPU oracle, bit for bit: the tile kernel (many rows), the operand-swapped kernel
(few rows) with every K-split mode, per-32 scale groups, padded buckets (live < M), odd N, strided outputs.  The cases
follow the reference's tests/test_cuda_gemm.py (shapes :24-29, poison-filled slots :82, rows >= live untouched :67)."""
import numpy as np
import pytest
import torch

import oracle
from prism_b200 import quant, w8a8
from util import bf16_from_bits, first_diff, n_rows, np_bits, rand_w8a8, same

pytestmark = pytest.mark.gpu

# (M, N, K, live)
SHAPES = [(8, 128, 256, 3), (1, 8192, 2560, 1), (16, 5120, 5120, 16), (64, 12352, 2560, 64), (64, 5120, 5120, 50),
          (33, 1000, 1024, 33), (100, 2560, 9216, 77), (256, 5120, 6144, 256), (384, 4608, 2560, 361),
          (130, 328, 400, 129),
          # one row with K % 256 == 0 against fewer than 9,472 weight rows: the CUDA-core kernel (cfg None / 1); N past
          # a whole warp of rows; the others stay on the tensor-core kernel
          (1, 5120, 5120, 1), (2, 1000, 1024, 2), (1, 34816, 512, 1), (1, 7168, 2560, 1), (1, 133, 256, 1),
          (1, 5120, 17408, 1), (1, 9000, 2560, 1)]


def run(dev, a, w, sa, sw, out, live, gk, epi, **kw):
    return w8a8.gemm(a.to(dev), sa.to(dev), w.to(dev), sw.to(dev), out, n_rows(live, dev), gk, epi=epi, **kw)


@pytest.mark.parametrize("M,N,K,live", SHAPES)
def test_gemm_one_group(dev, M, N, K, live):
    a, w, sa, sw = rand_w8a8(M, N, K, seed=M * 7 + N)
    an, wn, san, swn = a.numpy(), w.numpy(), sa.numpy(), sw.numpy()
    ref0 = oracle.w8a8_gemm(an, san, wn, swn, K, 0, live)
    base = torch.randn(M, N, generator=torch.Generator().manual_seed(1))
    ref1 = oracle.w8a8_gemm(an, san, wn, swn, K, 1, live, out=base.numpy())
    splits = [None, 1] + ([2, 3, 8] if M <= 64 else [2, 3])
    for split in splits:
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        run(dev, a, w, sa, sw, out, live, K, 0, cfg=split)
        assert same(out, bf16_from_bits(ref0)), ("bf16", split, first_diff(np_bits(out), ref0))
        res = base.to(dev)
        run(dev, a, w, sa, sw, res, live, K, 1, cfg=split)
        assert same(res, ref1), ("add", split, first_diff(res.cpu().numpy(), ref1))


@pytest.mark.parametrize("M,N,K,live", [(8, 128, 256, 3), (64, 5120, 6144, 64), (50, 5120, 17408, 47),
                                        (100, 5120, 17408, 77), (384, 2560, 2048, 361)])
def test_int32_slots_and_fold(dev, M, N, K, live):
    """gemm_i32 / deferred split-K: the slots' sum is the exact integer product, rows >= live keep the poison, and
    folding gives the unsplit residual add's bits (tests/test_cuda_gemm.py:175-225)."""
    a, w, sa, sw = rand_w8a8(M, N, K, seed=N + K)
    an, wn = a.numpy(), w.numpy()
    exact = oracle.w8a8_gemm(an, sa.numpy(), wn, sw.numpy(), K, 3, live)
    base = torch.randn(M, N, generator=torch.Generator().manual_seed(2))
    ref1 = oracle.w8a8_gemm(an, sa.numpy(), wn, sw.numpy(), K, 1, live, out=base.numpy())
    nr = n_rows(live, dev)
    ad, wd, sad, swd = a.to(dev), w.to(dev), sa.to(dev).view(-1), sw.to(dev).view(-1)
    for split in ([1, 2, 4] if M <= 64 else [1, 3]):
        slots = torch.full((4, M, N), -(1 << 30), dtype=torch.int32, device=dev)
        S = w8a8.gemm_i32(ad, sad, wd, swd, slots, nr, max_split=4, split=split)
        # many rows: K slices meet inside the kernel (workspace), one slot comes back
        assert S == (w8a8.effective_split(K, split) if M <= 64 else 1)
        tot = slots[:S, :live].sum(0, dtype=torch.int32)
        assert same(tot, exact[:live]), (split, first_diff(tot.cpu().numpy(), exact[:live]))
        assert bool((slots[:S, live:] == -(1 << 30)).all()) and bool((slots[S:] == -(1 << 30)).all())
        res = base.to(dev)
        quant.fold(res, slots, w8a8.Deferred(S, sad, swd), nr, M)
        assert same(res, ref1), (split, first_diff(res.cpu().numpy(), ref1))
    if M <= 64:
        # gemm() itself defers when given slots
        slots = torch.full((4, M, N), -(1 << 30), dtype=torch.int32, device=dev)
        res = base.to(dev)
        d = w8a8.gemm(ad, sad, wd, swd, res, nr, K, epi=1, slots=slots, cfg=4)
        assert isinstance(d, w8a8.Deferred) and d.n == w8a8.effective_split(K, 4)
        quant.fold(res, slots, d, nr, M)
        assert same(res, ref1)


@pytest.mark.parametrize("M,N,K,live", [(16, 5120, 5120, 16), (5, 256, 384, 4), (64, 1000, 1024, 61),
                                        (150, 512, 2560, 140), (3, 35840, 2048, 3),
                                        # the few-row kernel's corners: one 128-byte chunk of K; an odd number of
                                        # chunks (the last stage half fill); a last accumulator slot of one stage; row
                                        # blocks of 16 with one live row in the last; 4 / 8 / 16 rows per CTA; a K long
                                        # enough that the activation scales leave room for four stages only
                                        (1, 128, 128, 1), (16, 384, 640, 9), (17, 300, 1152, 17), (40, 5120, 5120, 33),
                                        (8, 5120, 13824, 8), (12, 640, 896, 12), (4, 256, 32768, 4), (2, 2560, 2560, 2)])
def test_gemm_q8_0_groups(dev, M, N, K, live):
    """gk = 32: Q8_0's own block scales, fp32 partial sums added in group order (kernels/w8a8.py:64-76).  The fifth
    case has more CTAs than SMs."""
    a, w, sa, sw = rand_w8a8(M, N, K, seed=K + M, groups=K // 32)
    ref0 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), 32, 0, live)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    run(dev, a, w, sa, sw, out, live, 32, 0)
    assert same(out, bf16_from_bits(ref0)), first_diff(np_bits(out), ref0)
    base = torch.randn(M, N, generator=torch.Generator().manual_seed(3))
    ref1 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), 32, 1, live, out=base.numpy())
    res = base.to(dev)
    run(dev, a, w, sa, sw, res, live, 32, 1)
    assert same(res, ref1), first_diff(res.cpu().numpy(), ref1)


def test_strided_output_and_determinism(dev):
    """out as a column slice of a wider buffer (engine/model.py:848), twice: same bits, neighbours untouched."""
    M, N, K = 48, 640, 1024
    a, w, sa, sw = rand_w8a8(M, N, K, seed=5)
    ref0 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), K, 0, M)
    for M2 in (M, 200):
        a2 = a if M2 == M else torch.cat([a, a, a, a, a[:8]])
        sa2 = sa if M2 == M else torch.cat([sa, sa, sa, sa, sa[:8]])
        wide = torch.full((M2, N + 200), 7.0, dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            run(dev, a2, w, sa2, sw, wide[:, 100:100 + N], M2, K, 0)
            assert same(wide[:M, 100:100 + N].contiguous(), bf16_from_bits(ref0))
            assert bool((wide[:, :100] == 7).all()) and bool((wide[:, 100 + N:] == 7).all())


def test_graph_replay_live_rows(dev):
    """One captured graph serves every live count: n_rows is read on the device (tests/test_cuda_gemm.py:149-169)."""
    M, N, K = 384, 1536, 2560
    a, w, sa, sw = rand_w8a8(M, N, K, seed=11)
    full = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), K, 0, M)
    ad, wd, sad, swd = a.to(dev), w.to(dev), sa.to(dev), sw.to(dev)
    nr = n_rows(M, dev)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(ad, sad, wd, swd, out, nr, K)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        w8a8.gemm(ad, sad, wd, swd, out, nr, K)
    for live in (1, 97, 128, 129, 300, 384):
        nr.fill_(live)
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert same(out[:live].contiguous(), bf16_from_bits(full[:live])), live
        assert live == M or not bool(out[live:].any())


def test_config0_synthetic(dev):
    """The reference's own CPU-runnable case: Q8_0 weights [5120, 5120] ~ N(0, 0.02^2), bf16 activations [16, 5120] with 8 outlier
    channels, per-token int8, per-32 block scales, bf16 out."""
    from prism_b200 import synth
    q8 = synth.q8_0(synth.weights(5120, 5120, synth.seed_w(0, 1)))
    x = synth.activations(16, 5120, synth.seed_x(0, 1, 16))
    wq, ws = w8a8.weight_from_q8(q8, 32)
    xq, xs = oracle.quant_rows(np_bits(x), 32)
    ref = oracle.w8a8_gemm(xq, xs, wq.numpy(), ws.numpy(), 32, 0)
    q, s = w8a8.quant_rows(x.to(dev), 32)
    assert same(q, xq) and same(s, xs)
    out = torch.zeros(16, 5120, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(q, s, wq.to(dev), ws.to(dev), out, n_rows(16, dev), 32)
    assert same(out, bf16_from_bits(ref)), first_diff(np_bits(out), ref)
    # the engine's mode: one scale per output channel (requantized), one per token
    wq1, ws1 = w8a8.weight_from_q8(q8, 5120)
    xq1, xs1 = oracle.quant_rows(np_bits(x))
    ref1 = oracle.w8a8_gemm(xq1, xs1, wq1.numpy(), ws1.numpy(), 5120, 0)
    q1 = torch.empty(16, 5120, dtype=torch.int8, device=dev)
    s1 = torch.empty(16, dtype=torch.float32, device=dev)
    quant.rows_q8(x.to(dev), None, q1, s1, n_rows(16, dev), 16)
    assert same(q1, xq1) and same(s1, xs1.reshape(-1))
    out1 = torch.zeros(16, 5120, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(q1, s1, wq1.to(dev), ws1.to(dev).view(-1), out1, n_rows(16, dev), 5120)
    assert same(out1, bf16_from_bits(ref1)), first_diff(np_bits(out1), ref1)


@pytest.mark.parametrize("M,N,K,live", [(512, 512, 1024, 512), (700, 1000, 2560, 650), (2048, 5120, 5120, 2048),
                                        (1300, 4608, 640, 1290)])
def test_gemm_cta_pairs(dev, M, N, K, live, monkeypatch):
    """The CTA-pair kernel (clusters of two, 256 x 256 tiles; PRISM_B200_PAIR=1 before the library's first GEMM): all
    three epilogues against the oracle bit for bit, partial tiles in M and N, rows >= live untouched.  Run in a child
    process so the switch is read afresh."""
    import os
    import subprocess
    import sys
    if os.environ.get("PRISM_B200_PAIR") != "1":
        env = dict(os.environ, PRISM_B200_PAIR="1")
        r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", __file__, "-k",
                            f"test_gemm_cta_pairs and {M}-{N}-{K}-{live}"], env=env, capture_output=True, text=True)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
        return
    a, w, sa, sw = rand_w8a8(M, N, K, seed=M + K)
    an, wn, san, swn = a.numpy(), w.numpy(), sa.numpy(), sw.numpy()
    ref0 = oracle.w8a8_gemm(an, san, wn, swn, K, 0, live)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    run(dev, a, w, sa, sw, out, live, K, 0)
    assert same(out, bf16_from_bits(ref0)), first_diff(np_bits(out), ref0)
    base = torch.randn(M, N, generator=torch.Generator().manual_seed(1))
    ref1 = oracle.w8a8_gemm(an, san, wn, swn, K, 1, live, out=base.numpy())
    res = base.to(dev)
    run(dev, a, w, sa, sw, res, live, K, 1)
    assert same(res, ref1), first_diff(res.cpu().numpy(), ref1)
    exact = oracle.w8a8_gemm(an, san, wn, swn, K, 3, live)
    slots = torch.full((1, M, N), -(1 << 30), dtype=torch.int32, device=dev)
    assert w8a8.gemm_i32(a.to(dev), sa.to(dev).view(-1), w.to(dev), sw.to(dev).view(-1), slots, n_rows(live, dev)) == 1
    assert same(slots[0, :live], exact[:live]) and bool((slots[0, live:] == -(1 << 30)).all())


@pytest.mark.parametrize("gk", [0, 32])
def test_programmatic_dependent_launch(dev, gk):
    """pdl=True: the GEMM may start while its producer (the quantizer of its input) still runs; the weights stream
    early, the activations are read after the producer completed.  Same bits, eagerly and in a replayed graph."""
    from prism_b200 import synth
    M, N, K = 16, 5120, 5120
    gkk = gk or K
    x = synth.activations(M, K, seed=77)
    w = torch.randint(-127, 128, (N, K), generator=torch.Generator().manual_seed(5), dtype=torch.int8)
    sw = torch.rand(N, K // gkk, generator=torch.Generator().manual_seed(6)) * 1e-3
    rq, rs = oracle.quant_rows(np_bits(x), gkk)
    ref = oracle.w8a8_gemm(rq, rs, w.numpy(), sw.numpy(), gkk, 0)
    xd, wd, swd = x.to(dev), w.to(dev), sw.to(dev)
    nr = n_rows(M, dev)
    q = torch.empty(M, K, dtype=torch.int8, device=dev)
    s = torch.empty(M, K // gkk, device=dev)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)

    def step():
        q.zero_()                                         # the producer really has to run before the GEMM reads q
        if gk:
            qq, ss = w8a8.quant_rows(xd, gk, nr)
            q.copy_(qq)
            s.copy_(ss)
        else:
            quant.rows_q8(xd, None, q, s.view(-1), nr, M)
        w8a8.gemm(q, s if gk else s.view(-1), wd, swd if gk else swd.view(-1), out, nr, gkk, pdl=True)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    assert same(out, bf16_from_bits(ref))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
            step()
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert same(out, bf16_from_bits(ref))


@pytest.mark.parametrize("M,N,K,split", [(16, 5120, 5120, 4), (1, 7168, 5120, 5), (64, 1000, 1024, 3), (8, 7168, 5120, 5)])
def test_q8_0_groups_split_k(dev, M, N, K, split):
    """gk = 32 with K splits (opt-in): slice sums are added in slice order - deterministic (two runs agree bit for
    bit) and within one bf16 step of the reference's unsplit group order; the fp32 residual add agrees to 1e-6."""
    a, w, sa, sw = rand_w8a8(M, N, K, seed=split, groups=K // 32)
    ref0 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), 32, 0)
    outs = []
    for _ in range(2):
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        run(dev, a, w, sa, sw, out, M, 32, 0, cfg=split)
        outs.append(out)
    assert same(outs[0], outs[1])
    # the slices' fp32 sums differ from the unsplit order by fp32 rounding of the partial sums (about 1e-5 absolute
    # here), which the bf16 store turns into at most one step except where the value itself is that small
    got = bf16_from_bits(np_bits(outs[0])).float().numpy()
    want = bf16_from_bits(ref0).float().numpy()
    assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 5e-5).all()
    assert (got != want).mean() < 0.01
    base = torch.randn(M, N, generator=torch.Generator().manual_seed(3))
    ref1 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), 32, 1, out=base.numpy())
    res = base.to(dev)
    w8a8._workspace(dev)[0].fill_(0xFF)          # a slice read before it was written would give NaN
    run(dev, a, w, sa, sw, res, M, 32, 1, cfg=split)
    assert np.allclose(res.cpu().numpy(), ref1, rtol=1e-5, atol=5e-5)


@pytest.mark.parametrize("M,N,K,live,gk", [(16, 512, 1024, 16, 64), (40, 200, 512, 37, 128), (5, 5120, 5120, 5, 256),
                                           (64, 1000, 2560, 61, 640), (150, 384, 1024, 140, 64), (33, 256, 3072, 33, 96)])
def test_gemm_any_group_size(dev, M, N, K, live, gk):
    """Scale groups of any multiple of 32 inputs that divides K (the reference's kernel takes any GK,
    kernels/w8a8.py:64-76): per group an exact integer sum, the scaled sums added in fp32 in group order."""
    a, w, sa, sw = rand_w8a8(M, N, K, seed=gk + M, groups=K // gk)
    ref0 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), gk, 0, live)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    run(dev, a, w, sa, sw, out, live, gk, 0)
    assert same(out, bf16_from_bits(ref0)), first_diff(np_bits(out), ref0)
    base = torch.randn(M, N, generator=torch.Generator().manual_seed(4))
    ref1 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), gk, 1, live, out=base.numpy())
    res = base.to(dev)
    run(dev, a, w, sa, sw, res, live, gk, 1)
    assert same(res, ref1), first_diff(res.cpu().numpy(), ref1)


@pytest.mark.parametrize("M,FF,K,live,bn", [(70, 256, 512, 66, 128), (20, 256, 256, 20, 64), (300, 640, 1024, 290, 128),
                                            (16, 17408 // 8, 5120, 16, 128)])
def test_gemm_swiglu_epilogue(dev, M, FF, K, live, bn):
    """epi 2: gate|up rows interleaved in tiles of bn, silu(gate) * up quantized per row and tile in the epilogue
    (kernels/w8a8.py:86-98).  The scales agree with the oracle to 1e-5, the int8 values within one step (the device's
    exp differs from libm's in the last bits); rows past the live count are untouched.  The output then feeds a down
    projection with gk = bn / 2, which must equal the oracle's product of the same int8 values bit for bit."""
    g = torch.Generator().manual_seed(M + FF)
    gate = torch.randint(-127, 128, (FF, K), generator=g, dtype=torch.int8)
    up = torch.randint(-127, 128, (FF, K), generator=g, dtype=torch.int8)
    gs, us = torch.rand(FF, generator=g) * 2e-3, torch.rand(FF, generator=g) * 2e-3
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    sa = torch.rand(M, generator=g) * 1e-2
    w = w8a8.interleave_gate_up(gate, up, bn)
    ws = w8a8.interleave_gate_up(gs.view(FF, 1), us.view(FF, 1), bn).view(-1)
    rq, rs = oracle.w8a8_swiglu_epi(a.numpy(), sa.numpy(), w.numpy(), ws.numpy(), bn, live)
    q = torch.full((M, FF), 77, dtype=torch.int8, device=dev)
    s = torch.full((M, 2 * FF // bn), -1.0, device=dev)
    w8a8.gemm(a.to(dev), sa.to(dev), w.to(dev), ws.to(dev), q, n_rows(live, dev), K, epi=2, outs=s, cfg=bn)
    torch.cuda.synchronize()
    qn, sn = q.cpu().numpy(), s.cpu().numpy()
    assert np.allclose(sn[:live], rs[:live], rtol=1e-5, atol=0)
    d = np.abs(qn[:live].astype(np.int32) - rq[:live].astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.01, (d.max(), (d != 0).mean())
    assert (qn[live:] == 77).all() and (sn[live:] == -1).all()
    # the consumer: a down projection whose activation scales are per bn / 2 inputs
    hb = bn // 2
    N2 = 256
    wd_ = torch.randint(-127, 128, (N2, FF), generator=g, dtype=torch.int8)
    wds = torch.rand(N2, FF // hb, generator=g) * 1e-3
    ref = oracle.w8a8_gemm(qn, sn, wd_.numpy(), wds.numpy(), hb, 0, live)
    out = torch.zeros(M, N2, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(q, s, wd_.to(dev), wds.to(dev), out, n_rows(live, dev), hb)
    assert same(out, bf16_from_bits(ref)), first_diff(np_bits(out), ref)


def test_l2_prefetch(dev):
    """The bulk L2 prefetch of weight ranges on a side stream: sizes that are not whole chunks, several tensors, then
    the GEMM that reads them - the bits do not change (a prefetch only moves cache lines)."""
    M, N, K = 16, 5120, 5120
    a, w, sa, sw = rand_w8a8(M, N, K, seed=9)
    ref0 = oracle.w8a8_gemm(a.numpy(), sa.numpy(), w.numpy(), sw.numpy(), K, 0, M)
    ad, wd, sad, swd = a.to(dev), w.to(dev), sa.to(dev).view(-1), sw.to(dev).view(-1)
    odd = torch.zeros(4096 * 3 + 48, dtype=torch.uint8, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        w8a8.l2_prefetch([wd, swd, odd], ctas=16)
        w8a8.l2_prefetch([wd])
    torch.cuda.current_stream().wait_stream(side)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    w8a8.gemm(ad, sad, wd, swd, out, n_rows(M, dev), K)
    torch.cuda.synchronize()
    assert same(out, bf16_from_bits(ref0))
    with pytest.raises(RuntimeError):
        w8a8.l2_prefetch([])
