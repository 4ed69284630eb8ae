"""MXFP4 on the GPU: the activation quantizer against the CPU oracle bit for bit (and the reference's golden vectors),
the GEMM against the dequantized product within 1e-3 relative Frobenius error (the reference's own test allows 2e-3,
tests/test_mxfp4.py:54-85), both epilogues, batch invariance (tests/test_mxfp4.py:88-102)."""
import os

import numpy as np
import pytest
import torch

import oracle
from prism_b200 import mxfp4, synth
from util import np_bits, same

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def quant_gpu(x, dev, inv=None):
    n, k = x.shape
    q = torch.zeros(n, k // 2, dtype=torch.uint8, device=dev)
    s = torch.zeros(n, k // 32, dtype=torch.uint8, device=dev)
    if inv is None:
        mxfp4.quantize_act(x.to(dev), q, s)
    else:
        mxfp4.quantize_act_scaled(x.to(dev), inv.to(dev), q, s)
    return q, s


def test_quantize_act_golden(dev):
    g = np.load(os.path.join(G, "mxfp4.npz"))
    xb = torch.from_numpy(g["act_bf16"].view(np.int16)).view(torch.bfloat16)
    q, s = quant_gpu(xb, dev)
    assert same(q, g["act_q_bf16"]) and same(s, g["act_s_bf16"])
    q, s = quant_gpu(torch.from_numpy(g["act_f32"]), dev)
    assert same(q, g["act_q_f32"]) and same(s, g["act_s_f32"])
    q, s = quant_gpu(xb, dev, torch.from_numpy(g["act_inv"]))
    assert same(q, g["act_q_scaled"]) and same(s, g["act_s_scaled"])


@pytest.mark.parametrize("n,k", [(7, 256), (33, 512), (128, 4096), (16, 5120), (3, 17408)])
def test_quantize_act_oracle(dev, n, k):
    x = synth.activations(n, k, seed=n + k)
    rq, rs = oracle.mxfp4_quant(np_bits(x))
    q, s = quant_gpu(x, dev)
    assert same(q, rq) and same(s, rs)
    dq = mxfp4.dequant_packed(q.cpu(), s.cpu())
    rel = (dq - x.float()).norm() / x.float().norm()
    assert rel < 0.2                                      # tests/test_mxfp4.py:41-51


def rel_fro(got, ref):
    return float(np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref))


def bf16_within_one_step(out, ref64):
    """A bf16 output against the float64 product rounded to bf16 (round to nearest even): equal, or its neighbour (fp32
    accumulation in another order can move a value across a rounding boundary).  The output's own rounding alone is
    1.1e-3 relative Frobenius error, so the bound on the bf16 path is this one, not a Frobenius figure."""
    want = torch.from_numpy(np.ascontiguousarray(ref64)).to(torch.bfloat16)
    got = out.detach().cpu()
    gi, wi = got.view(torch.int16).int(), want.view(torch.int16).int()
    tiny = (got.float().abs() < 1e-30) & (want.float().abs() < 1e-30)
    return bool((((gi - wi).abs() <= 1) | tiny).all())


@pytest.mark.parametrize("M,N,K", [(32, 512, 256), (257, 1024, 512), (16, 5120, 5120), (300, 1000, 2560),
                                   (1024, 4096, 4096), (1024, 4808, 512), (1000, 4664, 768), (2048, 5120, 1024)])
def test_gemm(dev, M, N, K):
    w = mxfp4.pack(synth.weights(N, K, seed=N + K))
    x = synth.activations(M, K, seed=M)
    q, s = quant_gpu(x, dev)
    wd = mxfp4.prepare(mxfp4.MX4(w.q.to(dev), w.s.to(dev), N, K))
    _, ref = oracle.mxfp4_gemm(q.cpu().numpy(), s.cpu().numpy(), w.q.numpy(), w.s.numpy())
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mxfp4.gemm(q, s, wd, out, M, epi=0)
    err0 = rel_fro(out.float().cpu().numpy(), ref)
    assert err0 < 2e-3, err0                              # the reference's own bound; the output's bf16 rounding dominates
    assert bf16_within_one_step(out, ref)                 # ... and every value is the rounded exact product or its neighbour
    h0 = torch.randn(M, N, generator=torch.Generator().manual_seed(1))
    h = h0.to(dev)
    mxfp4.gemm(q, s, wd, h, M, epi=1)
    err1 = rel_fro(h.cpu().numpy() - h0.numpy(), ref)
    assert err1 < 1e-3, err1                              # the fp32 accumulators against the float64 product


@pytest.mark.parametrize("M,N,K", [(16, 5120, 5120), (1, 1000, 2560), (64, 384, 4352), (100, 256, 1024)])
def test_gemm_k_split(dev, M, N, K):
    """K slices per tile, added in slice order by the tile's last CTA: the same tolerances as the unsplit product, the
    same bits on every run (a poisoned workspace in between), counters left zeroed."""
    from prism_b200 import w8a8
    w = mxfp4.pack(synth.weights(N, K, seed=N + K))
    q, s = quant_gpu(synth.activations(M, K, seed=M), dev)
    wd = mxfp4.prepare(mxfp4.MX4(w.q.to(dev), w.s.to(dev), N, K))
    _, ref = oracle.mxfp4_gemm(q.cpu().numpy(), s.cpu().numpy(), w.q.numpy(), w.s.numpy())
    ws, counters = w8a8._workspace(dev)
    for split in (2, 3, 5, "auto"):
        h0 = torch.randn(M, N, generator=torch.Generator().manual_seed(1))
        runs = []
        for rep in range(2):
            ws.fill_(0x7f)
            h = h0.to(dev)
            mxfp4.gemm(q, s, wd, h, M, epi=1, split=split)
            runs.append(h)
        assert same(runs[0], runs[1]), split
        assert rel_fro(runs[0].cpu().numpy() - h0.numpy(), ref) < 1e-5, split
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        mxfp4.gemm(q, s, wd, out, M, epi=0, split=split)
        assert rel_fro(out.float().cpu().numpy(), ref) < 2e-3, split
        assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("M,N,K", [(1, 5120, 5120), (2, 1000, 2560), (1, 133, 256), (2, 34816, 512), (4, 7168, 1024),
                                   (3, 300, 768)])
def test_gemv_rows(dev, M, N, K):
    """One to four rows on the CUDA-core kernel (exact integer block products, fp32 over the blocks) against the
    float64 product, both epilogues; deterministic; rows past M and columns past N untouched."""
    w = mxfp4.pack(synth.weights(N, K, seed=N + K))
    q, s = quant_gpu(synth.activations(M, K, seed=M + 7, outliers=K // 64), dev)
    wd = mxfp4.prepare(mxfp4.MX4(w.q.to(dev), w.s.to(dev), N, K))
    _, ref = oracle.mxfp4_gemm(q.cpu().numpy(), s.cpu().numpy(), w.q.numpy(), w.s.numpy())
    h0 = torch.randn(M + 1, N + 3, generator=torch.Generator().manual_seed(1))
    runs = []
    for rep in range(2):
        h = h0.to(dev)
        mxfp4.gemv(q, s, wd, h[:M, :N], M, epi=1)
        runs.append(h)
    assert same(runs[0], runs[1])
    got = runs[0].cpu().numpy()
    assert rel_fro(got[:M, :N] - h0.numpy()[:M, :N], ref) < 1e-5
    assert np.array_equal(got[M:], h0.numpy()[M:]) and np.array_equal(got[:, N:], h0.numpy()[:, N:])
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mxfp4.gemv(q, s, wd, out, M, epi=0)
    assert rel_fro(out.float().cpu().numpy(), ref) < 2e-3 and bf16_within_one_step(out, ref)
    if M == 1:                                            # split="auto" routes one row against few weight rows here
        auto = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        mxfp4.gemm(q, s, wd, auto, M, epi=0, split="auto")
        assert rel_fro(auto.float().cpu().numpy(), ref) < 2e-3
    # and close to the tensor-core kernel's bits: the same exact block products, another order of fp32 additions
    out_tc = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mxfp4.gemm(q, s, wd, out_tc, M, epi=0)
    assert rel_fro(out.float().cpu().numpy(), out_tc.float().cpu().numpy().astype(np.float64)) < 2e-3


def test_gemm_fp32_path_tight(dev):
    """Against the float64 product the fp32-accumulated result is within 1e-5 (no operand rounding happens inside the
    MMA: e2m1 products and power-of-two scales are exact; only the fp32 sums round)."""
    M, N, K = 64, 256, 1024
    w = mxfp4.pack(synth.weights(N, K, seed=3))
    q, s = quant_gpu(synth.activations(M, K, seed=4), dev)
    wd = mxfp4.prepare(mxfp4.MX4(w.q.to(dev), w.s.to(dev), N, K))
    _, ref = oracle.mxfp4_gemm(q.cpu().numpy(), s.cpu().numpy(), w.q.numpy(), w.s.numpy())
    h = torch.zeros(M, N, device=dev)
    mxfp4.gemm(q, s, wd, h, M, epi=1)
    assert rel_fro(h.cpu().numpy(), ref) < 1e-5


def test_batch_invariance(dev):
    M, N, K = 64, 1024, 512
    w = mxfp4.pack(synth.weights(N, K, seed=5))
    wd = mxfp4.prepare(mxfp4.MX4(w.q.to(dev), w.s.to(dev), N, K))
    q, s = quant_gpu(synth.activations(M, K, seed=6), dev)
    out64 = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mxfp4.gemm(q, s, wd, out64, M)
    out32 = torch.zeros(32, N, dtype=torch.bfloat16, device=dev)
    mxfp4.gemm(q[:32].contiguous(), s[:32].contiguous(), wd, out32, 32)
    assert same(out64[:32].contiguous(), out32)
    big = torch.zeros(300, N, dtype=torch.bfloat16, device=dev)
    q3 = torch.cat([q] * 5)[:300].contiguous()
    s3 = torch.cat([s] * 5)[:300].contiguous()
    mxfp4.gemm(q3, s3, wd, big, 300)
    assert same(big[:64].contiguous(), out64) and same(big[256:300].contiguous(), out64[:44].contiguous())


def test_wide_tiles_same_bits(dev):
    """Enough tiles for the 128 x 256 kernel (at least one per SM): every row's bits equal the 128 x 128 kernel's (which
    runs when the same rows come in a small batch) - one accumulator over all of K either way."""
    M, N, K = 2048, 5120, 1024
    w = mxfp4.pack(synth.weights(N, K, seed=3))
    wd = mxfp4.prepare(mxfp4.MX4(w.q.to(dev), w.s.to(dev), N, K))
    q, s = quant_gpu(synth.activations(M, K, seed=4), dev)
    big = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mxfp4.gemm(q, s, wd, big, M)
    for r0 in (0, 900, 1984):
        small = torch.zeros(64, N, dtype=torch.bfloat16, device=dev)
        mxfp4.gemm(q[r0:r0 + 64].contiguous(), s[r0:r0 + 64].contiguous(), wd, small, 64)
        assert same(big[r0:r0 + 64].contiguous(), small)
