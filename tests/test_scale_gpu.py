"""Parity at the benchmarked sizes: M = 2048 and 8192 rows (full, and with three rows of the bucket not live) on the
27B-class layer shapes - q|k|v [7168, 5120], o [5120, 5120], gate|up [34816, 5120], down [5120, 17408] - for W8A8
(bf16 store, fp32 residual add, int32 sums), W4A8 (the Q4_K_M assignment) and MXFP4.

The CPU oracle cannot finish a whole 8192-row product in seconds, so, following the reference's own test of padded
buckets (tests/test_cuda_gemm.py:24-29,56-67), it is run on 64 seeded rows - one in every 128-row tile the kernel
forms, each at a different offset inside its tile, plus the last live row - over ALL output columns, bit for bit.  For
W8A8 the whole output is also compared on the GPU with the exact integer product (torch._int_mm) pushed through the same
three roundings as separate torch operations: every tile of every wave, the weight-tiles-fastest order of the down
projection at 8192 rows and the copy-engine residual add included."""
import numpy as np
import pytest
import torch

import oracle
from prism_b200 import gguf_weights as GW
from prism_b200 import mxfp4, quant, w4a8, w8a8
from util import n_rows

pytestmark = pytest.mark.gpu

SHAPES = {"qkv": (7168, 5120), "o": (5120, 5120), "gate_up": (34816, 5120), "down": (5120, 17408)}
POISON_BF16, POISON_I32 = 7.0, -(1 << 30)


def sample_rows(M, live):
    """64 rows: tile i % tiles at offset (37 i + 5) % 128 (37 is odd: 63 different offsets), and the last live row."""
    tiles = (M + 127) // 128
    rows = {min(live - 1, (i % tiles) * 128 + (37 * i + 5) % 128) for i in range(63)}
    rows.add(live - 1)
    return np.array(sorted(rows))


def operands(N, K, M, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    sa = torch.rand(M, generator=g) * 1e-2 + 1e-4
    sw = torch.rand(N, generator=g) * 1e-3 + 1e-5
    return a, w, sa, sw


@pytest.mark.parametrize("M", [2048, 8192])
@pytest.mark.parametrize("name", list(SHAPES))
def test_w8a8_at_scale(dev, name, M):
    N, K = SHAPES[name]
    a, w, sa, sw = operands(N, K, M, seed=M + N)
    ad, wd, sad, swd = a.to(dev), w.to(dev), sa.to(dev), sw.to(dev)
    base = torch.randn(M, N, generator=torch.Generator(device=dev).manual_seed(7), device=dev)
    # whole-matrix checker on the GPU: exact integer product, then the contract's roundings one torch op at a time
    try:
        exact = torch._int_mm(ad, wd.t())
    except Exception as e:                                  # noqa: BLE001
        exact = None
        print(f"torch._int_mm unavailable ({e}): whole-matrix comparison skipped, sampled rows only")
    for live in (M, M - 3):
        rows = sample_rows(M, live)
        an, san = a[rows].numpy(), sa[rows].view(-1, 1).numpy()
        wn, swn = w.numpy(), sw.view(-1, 1).numpy()
        nr = n_rows(live, dev)
        want0 = oracle.w8a8_gemm(an, san, wn, swn, K, 0)
        out = torch.full((M, N), POISON_BF16, dtype=torch.bfloat16, device=dev)
        w8a8.gemm(ad, sad, wd, swd, out, nr, K, epi=0)
        got0 = out[torch.from_numpy(rows).to(dev)].cpu().view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(got0, want0), (name, M, live, "bf16", np.argwhere(got0 != want0)[:3])
        assert bool((out[live:] == POISON_BF16).all())
        want1 = oracle.w8a8_gemm(an, san, wn, swn, K, 1, out=base[torch.from_numpy(rows).to(dev)].cpu().numpy())
        res = base.clone()
        w8a8.gemm(ad, sad, wd, swd, res, nr, K, epi=1)
        got1 = res[torch.from_numpy(rows).to(dev)].cpu().numpy()
        assert np.array_equal(got1.view(np.uint32), want1.view(np.uint32)), (name, M, live, "add")
        assert torch.equal(res[live:], base[live:])
        want3 = oracle.w8a8_gemm(an, san, wn, swn, K, 3)
        slots = torch.full((1, M, N), POISON_I32, dtype=torch.int32, device=dev)
        assert w8a8.gemm_i32(ad, sad, wd, swd, slots, nr, max_split=1) == 1
        got3 = slots[0][torch.from_numpy(rows).to(dev)].cpu().numpy()
        assert np.array_equal(got3, want3), (name, M, live, "int32")
        assert bool((slots[0, live:] == POISON_I32).all())
        if exact is not None:
            assert torch.equal(slots[0, :live], exact[:live]), (name, M, live, "int32 whole matrix")
            v = (exact[:live].float() * sad[:live, None]) * swd[None, :]
            assert torch.equal(out[:live].view(torch.int16), v.to(torch.bfloat16).view(torch.int16)), (name, M, live)
            assert torch.equal(res[:live], base[:live] + v), (name, M, live, "add whole matrix")
            del v
        del out, res, slots


@pytest.mark.parametrize("name,M", [("o", 2048), ("qkv", 2048), ("down", 256), ("o", 8192)])
def test_w8a8_q8_0_groups_at_scale(dev, name, M):
    """Q8_0's own scale per 32 inputs on both operands (config 1 run with GK = 32) at prefill row counts: the fp32 sum
    in group order (kernels/w8a8.py:64-76), row blocks of 32 per CTA.  64 sampled rows against the oracle, bf16 store
    and fp32 residual add, live < M; rows past live keep their poison."""
    N, K = SHAPES[name]
    G = K // 32
    g = torch.Generator().manual_seed(M + N + 1)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    sa = torch.rand(M, G, generator=g) * 1e-2 + 1e-4
    sw = torch.rand(N, G, generator=g) * 1e-3 + 1e-5
    ad, wd, sad, swd = a.to(dev), w.to(dev), sa.to(dev), sw.to(dev)
    base = torch.randn(M, N, generator=torch.Generator(device=dev).manual_seed(9), device=dev)
    for live in (M, M - 3):
        rows = sample_rows(M, live)
        idx = torch.from_numpy(rows).to(dev)
        an, san = a[rows].numpy(), sa[rows].numpy()
        nr = n_rows(live, dev)
        want0 = oracle.w8a8_gemm(an, san, w.numpy(), sw.numpy(), 32, 0)
        out = torch.full((M, N), POISON_BF16, dtype=torch.bfloat16, device=dev)
        w8a8.gemm(ad, sad, wd, swd, out, nr, 32, epi=0)
        got0 = out[idx].cpu().view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(got0, want0), (name, M, live, "bf16", np.argwhere(got0 != want0)[:3])
        assert bool((out[live:] == POISON_BF16).all())
        want1 = oracle.w8a8_gemm(an, san, w.numpy(), sw.numpy(), 32, 1, out=base[idx].cpu().numpy())
        res = base.clone()
        w8a8.gemm(ad, sad, wd, swd, res, nr, 32, epi=1)
        assert np.array_equal(res[idx].cpu().numpy().view(np.uint32), want1.view(np.uint32)), (name, M, live, "add")
        assert torch.equal(res[live:], base[live:])
        del out, res


def random_kquant(kind, n, k, seed):
    """Valid random k-quant blocks (any valid block is a valid input): random quants and 6-bit / int8 sub-block scales,
    fp16 d / dmin of the magnitude N(0, 0.02^2) weights give."""
    g = torch.Generator().manual_seed(seed)
    nb = n * (k // 256)
    if kind == "q4k":
        raw = torch.randint(0, 256, (nb, 144), generator=g, dtype=torch.uint8)
        d = (torch.rand(nb, generator=g) * 1e-4 + 5e-5).to(torch.float16)
        dm = (torch.rand(nb, generator=g) * 1e-3 + 1e-4).to(torch.float16)
        raw[:, 0:2] = d.view(torch.uint8).view(nb, 2)
        raw[:, 2:4] = dm.view(torch.uint8).view(nb, 2)
        return GW.KQuant(raw.view(n, k // 256, 144).contiguous(), GW.GGML_Q4_K, k)
    raw = torch.randint(0, 256, (nb, 210), generator=g, dtype=torch.uint8)
    d = (torch.rand(nb, generator=g) * 2e-5 + 1e-5).to(torch.float16)
    raw[:, 208:210] = d.view(torch.uint8).view(nb, 2)
    return GW.KQuant(raw.view(n, k // 256, 210).contiguous(), GW.GGML_Q6_K, k)


# the Q4_K_M assignment: q, k rows Q4_K and v rows Q6_K fused in one projection; o and gate|up Q4_K; down Q6_K.  gate|up
# is cut to a quarter of its rows here: the kernel's grid is one CTA per 128 x 64 tile, more columns add no code path.
W4_SEGS = {"qkv": [("q4k", 6144), ("q6k", 1024)], "o": [("q4k", 5120)], "gate_up": [("q4k", 8704)], "down": [("q6k", 5120)]}


@pytest.mark.parametrize("M", [2048, 8192])
@pytest.mark.parametrize("name", list(W4_SEGS))
def test_w4a8_at_scale(dev, name, M):
    K = SHAPES[name][1]
    kqs = [random_kquant(kind, n, K, seed=n + i) for i, (kind, n) in enumerate(W4_SEGS[name])]
    cpu = [w4a8.repack(kq) for kq in kqs]
    segs = w4a8.segments(kqs, dev)
    N = w4a8.seg_width(segs)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16)
    x[:, ::701] *= 20
    xd = x.to(dev)
    q = torch.empty(M, K, dtype=torch.int8, device=dev)
    a = torch.empty(K // 256, M, device=dev)
    xs = torch.empty(K // 256, M, 16, dtype=torch.int8, device=dev)
    quant.rows_g(xd, q, a, xs, n_rows(M, dev), M)
    base = torch.randn(M, N, generator=torch.Generator(device=dev).manual_seed(9), device=dev)
    for live in (M, M - 3):
        rows = sample_rows(M, live)
        rq, ra, rxs = oracle.quant_g(x[rows].view(torch.int16).numpy().view(np.uint16))
        rt = torch.from_numpy(rows).to(dev)
        assert np.array_equal(q[rt].cpu().numpy(), rq)       # the producer at this size feeds the same bytes
        nr = n_rows(live, dev)
        out = torch.full((M, N), POISON_BF16, dtype=torch.bfloat16, device=dev)
        w4a8.gemm_segs(q, a, xs, segs, out, nr)
        res = base.clone()
        w4a8.gemm_segs(q, a, xs, segs, res, nr, epi=1)
        off = 0
        for w in cpu:
            g = lambda t: None if t is None else t.numpy()  # noqa: E731
            want0 = oracle.w4a8_gemm(rq, ra, rxs, w.kind, g(w.q), g(w.sc), g(w.mn), g(w.d), g(w.dm), epi=0)
            got0 = out[rt, off:off + w.n].cpu().view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(got0, want0), (name, M, live, w.kind, np.argwhere(got0 != want0)[:3])
            want1 = oracle.w4a8_gemm(rq, ra, rxs, w.kind, g(w.q), g(w.sc), g(w.mn), g(w.d), g(w.dm), epi=1,
                                     out=base[rt, off:off + w.n].cpu().numpy())
            got1 = res[rt, off:off + w.n].cpu().numpy()
            assert np.array_equal(got1.view(np.uint32), want1.view(np.uint32)), (name, M, live, w.kind, "add")
            off += w.n
        assert bool((out[live:] == POISON_BF16).all()) and torch.equal(res[live:], base[live:])


MX_ROWS = {"qkv": 7168, "o": 5120, "gate_up": 8704, "down": 5120}       # gate|up cut as above


@pytest.mark.parametrize("M", [2048, 8192])
@pytest.mark.parametrize("name", list(MX_ROWS))
def test_mxfp4_at_scale(dev, name, M):
    """bf16 outputs against the float64 product of the dequantized operands rounded to bf16: equal or one bf16 step
    apart (fp32 accumulation in another order can move a value across a rounding boundary), and within 1e-3 relative
    Frobenius error before rounding on the fp32 path."""
    N, K = MX_ROWS[name], SHAPES[name][1]
    g = torch.Generator().manual_seed(N + M)
    wq = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    ws = torch.randint(117, 123, (N, K // 32), generator=g, dtype=torch.uint8)
    w = mxfp4.prepare(mxfp4.MX4(wq.to(dev), ws.to(dev), N, K))
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    x[:, ::701] *= 20
    aq = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
    as_ = torch.empty(M, K // 32, dtype=torch.uint8, device=dev)
    mxfp4.quantize_act(x.to(dev), aq, as_)
    for live in (M, M - 3):
        rows = sample_rows(M, live)
        rt = torch.from_numpy(rows).to(dev)
        _, sums = oracle.mxfp4_gemm(aq[rt].cpu().numpy(), as_[rt].cpu().numpy(), wq.numpy(), ws.numpy())
        out = torch.full((M, N), POISON_BF16, dtype=torch.bfloat16, device=dev)
        mxfp4.gemm(aq, as_, w, out, live, epi=0)
        got = out[rt].cpu()
        want = torch.from_numpy(sums).to(torch.bfloat16)                 # float64 -> bf16, round to nearest even
        gi, wi = got.view(torch.int16).int(), want.view(torch.int16).int()
        # neighbours in bf16 have adjacent bit patterns (same sign); a value next to zero may flip sign
        apart = (gi - wi).abs()
        near_zero = (got.float().abs() < 1e-30) & (want.float().abs() < 1e-30)
        assert bool(((apart <= 1) | near_zero).all()), (name, M, live, int(apart.max()))
        print(f"mxfp4 {name} M={M} live={live}: {(apart == 0).float().mean():.4f} of sampled bf16 outputs bit-equal")
        assert bool((out[live:] == POISON_BF16).all())
        res = torch.zeros(M, N, device=dev)
        mxfp4.gemm(aq, as_, w, res, live, epi=1)
        err = np.linalg.norm(res[rt].cpu().double().numpy() - sums) / np.linalg.norm(sums)
        assert err < 1e-3, (name, M, live, err)
