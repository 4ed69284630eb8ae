"""The CPU oracle against the golden vectors produced by the reference's own CPU-runnable code
(tests/golden/make_golden.py) and against its literal known-answer vectors.  CPU only."""
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import emulation

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return np.load(os.path.join(G, name))


def test_w4a8_quantize_ref():
    g = load("w4a8.npz")
    q, a, xs = oracle.quant_g(g["x"])
    assert np.array_equal(q, g["xq"]) and np.array_equal(a, g["a"]) and np.array_equal(xs, g["xs"])
    sums = xs.transpose(1, 0, 2).reshape(5, -1, 2, 8).astype(np.int32)
    assert np.array_equal((sums[:, :, 0] + 64 * sums[:, :, 1]).reshape(5, -1), g["sums"])


@pytest.mark.parametrize("kind,tag", [("q4k", "4"), ("q6k", "6")])
def test_w4a8_gemm_ref(kind, tag):
    """orc_w4a8_gemm (hardware fmaf) == the reference's gemm_ref (its float64 emulation of a fused multiply-add)."""
    g = load("w4a8.npz")
    mn = g["mn4"] if kind == "q4k" else None
    dm = g["dm4"] if kind == "q4k" else None
    base = np.zeros((5, 24), np.float32)
    y = oracle.w4a8_gemm(g["xq"], g["a"], g["xs"], kind, g[f"q{tag}"], g[f"sc{tag}"], mn, g[f"d{tag}"], dm, epi=1,
                         out=base)
    assert np.array_equal(y.view(np.uint32), g[f"y{tag}"].view(np.uint32))
    yb = oracle.w4a8_gemm(g["xq"], g["a"], g["xs"], kind, g[f"q{tag}"], g[f"sc{tag}"], mn, g[f"d{tag}"], dm, epi=0)
    assert np.array_equal(yb, oracle.bf16_bits(g[f"y{tag}"]))


def test_fma_emulation_is_fmaf():
    """The reference's fma32 (w4a8.py:164-174) equals a hardware single-rounding fma on its own samples."""
    g = load("w4a8.npz")
    got = np.array([np.float32(np.float64(a) * np.float64(b) + np.float64(c)) for a, b, c in
                    zip(g["fa"][:64], g["fb"][:64], g["fc"][:64])])          # double rounding differs rarely: only a hint
    import ctypes
    libm = ctypes.CDLL("libm.so.6")
    libm.fmaf.restype = ctypes.c_float
    libm.fmaf.argtypes = [ctypes.c_float] * 3
    hw = np.array([libm.fmaf(float(a), float(b), float(c)) for a, b, c in zip(g["fa"], g["fb"], g["fc"])], np.float32)
    assert np.array_equal(hw.view(np.uint32), g["fma"].view(np.uint32))
    assert np.mean(got == g["fma"][:64]) > 0.9


def test_mxfp4_activation_quant():
    g = load("mxfp4.npz")
    for tag in ("bf16", "f32"):
        q, s = oracle.mxfp4_quant(g[f"act_{tag}"])
        assert np.array_equal(s, g[f"act_s_{tag}"]), tag
        assert np.array_equal(q, g[f"act_q_{tag}"]), tag
    q, s = oracle.mxfp4_quant(g["act_bf16"], inv=g["act_inv"])
    assert np.array_equal(s, g["act_s_scaled"]) and np.array_equal(q, g["act_q_scaled"])


def test_mxfp4_weight_rule_and_grid():
    """The exact exponent rule equals numpy's ceil(log2(amax / 6)) on the reference's packed weights, and the
    known-answer grid of tests/test_mxfp4.py:34-38 survives quantize -> dequantize."""
    g = load("mxfp4.npz")
    q, s = oracle.mxfp4_quant(g["w"], neg_zero=False)
    assert np.array_equal(s, g["s_max"]) and np.array_equal(q, g["q_max"])
    q, s = oracle.mxfp4_quant(g["grid"], neg_zero=False)
    assert np.array_equal(q, g["grid_q"]) and np.array_equal(s, g["grid_s"])
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    deq = np.empty((1, 32), np.float32)
    deq[:, 0::2], deq[:, 1::2] = lut[q & 15], lut[q >> 4]
    deq *= np.exp2(s.astype(np.int32) - 127).astype(np.float32)
    assert np.abs(deq - g["grid"]).max() < 1e-6
    assert np.array_equal(deq, g["grid_deq"])


def test_mxfp4_gemm_is_dequantized_product():
    g = load("mxfp4.npz")
    aq, a_s = g["act_q_bf16"][:, :128], g["act_s_bf16"][:, :8]
    _, acc = oracle.mxfp4_gemm(aq, a_s, g["q_max"], g["s_max"])
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], np.float64)

    def deq(q, s):
        o = np.empty((q.shape[0], q.shape[1] * 2))
        o[:, 0::2], o[:, 1::2] = lut[q & 15], lut[q >> 4]
        return (o.reshape(q.shape[0], -1, 32) * np.exp2(s.astype(np.float64) - 127)[..., None]).reshape(q.shape[0], -1)
    assert np.array_equal(deq(g["q_max"], g["s_max"]).astype(np.float32), g["deq_max"])
    ref = deq(aq, a_s) @ deq(g["q_max"], g["s_max"]).T
    assert np.allclose(acc, ref, rtol=1e-12, atol=0)


def test_w8a8_gemm_against_float64():
    """The bound the reference's own test uses (tests/test_cuda_gemm.py:50,66-67,95): bf16 store within 8e-3 and the
    fp32 residual add within 1e-4 of the float64 product; int32 sums exact; per-32 groups likewise."""
    rng = np.random.default_rng(0)
    M, N, K = 9, 40, 512
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    for G in (1, K // 32):
        sa = (rng.random((M, G)) * 1e-2).astype(np.float32)
        sw = (rng.random((N, G)) * 1e-3).astype(np.float32)
        ref = np.zeros((M, N))
        for g in range(G):
            ks = slice(g * K // G, (g + 1) * K // G)
            ref += (a[:, ks].astype(np.float64) @ w[:, ks].astype(np.float64).T) * sa[:, g:g + 1] * sw[:, g][None]
        o0 = oracle.bf16_to_f32(oracle.w8a8_gemm(a, sa, w, sw, K // G, 0, live=7))
        rel = np.abs(o0[:7] - ref[:7]) / np.maximum(np.abs(ref[:7]), 1e-2)
        assert rel.max() < 8e-3 and not o0[7:].any()
        o1 = oracle.w8a8_gemm(a, sa, w, sw, K // G, 1, out=np.ones((M, N), np.float32))
        assert (np.abs(o1 - 1 - ref) / np.maximum(np.abs(ref), 1e-2)).max() < 1e-4
    exact = oracle.w8a8_gemm(a, sa, w, sw, K, 3)
    assert np.array_equal(exact, a.astype(np.int64) @ w.astype(np.int64).T)
    # fold of K-split int32 slots == the unsplit residual add
    sa1, sw1 = sa[:, :1].copy(), sw[:, :1].copy()
    halves = np.stack([a[:, :256].astype(np.int32) @ w[:, :256].astype(np.int32).T,
                       a[:, 256:].astype(np.int32) @ w[:, 256:].astype(np.int32).T])
    h = rng.standard_normal((M, N)).astype(np.float32)
    assert np.array_equal(oracle.fold(h, halves, sa1[:, 0], sw1[:, 0]),
                          oracle.w8a8_gemm(a, sa1, w, sw1, K, 1, out=h))


def test_quant_rows_matches_torch_division():
    """IEEE contract: the oracle's per-token quantizer equals torch's true division / round-half-even."""
    x = torch.randn(7, 640, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    bits = x.view(torch.int16).numpy().view(np.uint16)
    q, s = oracle.quant_rows(bits)
    xf = x.float()
    sc = xf.abs().amax(1).clamp_min(1e-10) / torch.full((7,), 127.0)
    assert np.array_equal(s[:, 0], sc.numpy())
    assert np.array_equal(q, torch.round(xf / sc[:, None]).to(torch.int8).numpy())
    q32, s32 = oracle.quant_rows(bits, 32)
    sg = xf.view(7, 20, 32).abs().amax(-1).clamp_min(1e-10) / torch.full((7, 20), 127.0)
    assert np.array_equal(s32, sg.numpy())


def test_cpu_emulation_fake_quantizers():
    g = load("sims.npz")
    x = torch.from_numpy(g["x"])
    assert np.array_equal(emulation.int8_rows(x).numpy(), g["int8_rows"])
    assert np.array_equal(emulation.int8_groups(32)(x).numpy(), g["int8_g32"])


def test_norm_q8_against_float64():
    """The norm_q8 restatement against the same formula in float64 (kernels/quant.py:166-170): at most one int8 step
    apart on rare values, scales to 1e-6; the deferred add inside it is the fold's."""
    rng = np.random.default_rng(5)
    T, HID = 6, 1024
    h = (rng.standard_normal((T, HID)) * 2).astype(np.float32)
    w = (rng.random(HID) + 0.5).astype(np.float32)
    q, s = oracle.norm_q8(h.copy(), w, 1e-6)
    h64 = h.astype(np.float64)
    y = h64 / np.sqrt((h64 * h64).mean(1, keepdims=True) + 1e-6) * w
    scale = np.maximum(np.abs(y).max(1), 1e-10) / 127.0
    assert np.allclose(s, scale, rtol=1e-6)
    want = np.rint(y / scale[:, None])
    assert np.abs(q - want).max() <= 1 and (q != want).mean() < 1e-3
    slots = rng.integers(-10 ** 6, 10 ** 6, (2, T, HID), dtype=np.int32)
    sa, sw = (rng.random(T) * 1e-2).astype(np.float32), (rng.random(HID) * 1e-3).astype(np.float32)
    h2 = h.copy()
    oracle.norm_q8(h2, w, 1e-6, parts=slots, psa=sa, psw=sw)
    assert np.array_equal(h2, oracle.fold(h.copy(), slots, sa, sw))


def test_gated_norm_q8_against_float64():
    rng = np.random.default_rng(9)
    T, HV, D, P, z_off = 4, 6, 128, 1000, 40
    o = (rng.standard_normal((T, HV * D)) * 2).astype(np.float32)
    z32 = (rng.standard_normal((T, P)) * 1.5).astype(np.float32)
    zb = oracle.bf16_bits(z32)
    w = (rng.random(D) + 0.5).astype(np.float32)
    inv = np.exp(rng.standard_normal(HV * D) * 0.1).astype(np.float32)
    q, s = oracle.gated_norm_q8(o, zb, z_off, w, inv, HV, D, 1e-6)
    o64 = o.astype(np.float64).reshape(T, HV, D)
    z = oracle.bf16_to_f32(zb).astype(np.float64)[:, z_off:z_off + HV * D].reshape(T, HV, D)
    y = o64 / np.sqrt((o64 * o64).mean(2, keepdims=True) + 1e-6) * w * (z / (1 + np.exp(-z))) * inv.reshape(HV, D)
    y = y.reshape(T, -1)
    scale = np.maximum(np.abs(y).max(1), 1e-10) / 127.0
    assert np.allclose(s, scale, rtol=1e-5)
    want = np.rint(y / scale[:, None])
    assert np.abs(q - want).max() <= 1 and (q != want).mean() < 5e-3
