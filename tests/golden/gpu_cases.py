"""Seeded inputs of the GPU-recorded golden file (gpu_ref.npz): one definition shared by the script that records the
reference's own Triton kernels on a B200 (make_golden_gpu.py) and by the tests that replay the same inputs through the
CPU oracle and through this library's CUDA kernels.  Only the outputs are stored in the fixture; the inputs are drawn
here from torch's CPU generator, which gives the same values on every machine of the same torch build.

Value distributions follow the benchmark configs: weights N(0, 0.02^2) through Q8_0, activations N(0, 1) with eight
outlier columns scaled by 20 (the pattern of the reference's tests/test_w4a8.py:26-30)."""
import numpy as np
import torch

# name -> (M, N, K, live, gk, epilogues); gk == 0 stands for "one group over all of K"
GEMM_CASES = {
    "few_oneK": (48, 384, 1024, 45, 0, (0, 1, 3)),
    "many_oneK_oddN": (130, 328, 512, 129, 0, (0, 1, 3)),
    "few_gk32": (16, 256, 1024, 16, 32, (0, 1)),
    "few_gk32_oddN": (40, 200, 512, 37, 32, (0, 1)),
    "few_gk128": (40, 200, 512, 37, 128, (0, 1)),
    "few_gk64": (24, 256, 512, 24, 64, (0,)),
    "many_gk32": (200, 512, 1024, 197, 32, (0,)),
}
# name -> (M, FF, K, live, BN): the fused SwiGLU epilogue on interleaved gate|up weights (tile of BN weight rows)
SWIGLU_EPI_CASES = {
    "epi2_bn128": (70, 256, 512, 66, 128),
    "epi2_bn64": (20, 192, 256, 20, 64),
}
# name -> (T, K, live, with_inv)
ROWS_CASES = {
    "rows_5120": (24, 5120, 21, False),
    "rows_5120_inv": (24, 5120, 24, True),
    "rows_17408": (6, 17408, 6, False),
}
# name -> (T, FF, live, with_inv)
SWIGLU_CASES = {
    "swiglu_17408": (6, 17408, 5, False),
    "swiglu_1024_inv": (20, 1024, 20, True),
}
# name -> (T, HID, live, n_parts, gather)
NORM_CASES = {
    "norm_plain": (16, 5120, 14, 0, False),
    "norm_pending": (16, 5120, 16, 2, False),
    "norm_gather": (8, 2560, 8, 0, True),
}
FOLD_CASE = (16, 5120, 13, 3)                 # rows, HID, live, S
GROUPS_CASE = (16, 1024, 32)                  # M, K, gk   (w8a8.quant_rows)
GATED_CASE = (8, 48, 128, 6)                  # T, HV, D, live
HEAD_CASE = (4, 5120, 512, 3)                 # B, HID, N, live   (head_quant, then head_q8 on N weight rows)
MXFP4_CASE = (64, 256, 1024)                  # M, N, K
EPS = 1e-6


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def activations(rows, K, seed, dtype=torch.bfloat16):
    g = _gen(seed)
    x = torch.randn(rows, K, generator=g)
    idx = torch.randint(0, K, (8,), generator=g)
    x[:, idx] *= 20
    return x.to(dtype)


def inv_factors(K, seed):
    return torch.exp(torch.randn(K, generator=_gen(seed)) * 0.1)


def q8_0(w):
    """ggml's Q8_0 rule on fp32 [N, K]: d = max|w| / 127 per 32, q = round(w / d) with the fp32 d, d stored as fp16."""
    N, K = w.shape
    g = w.view(N, K // 32, 32)
    d = g.abs().amax(-1) / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(g * inv[..., None]).clamp(-127, 127).to(torch.int8).view(N, K)
    return q.contiguous(), d.to(torch.float16).contiguous()


def regroup(q, d16, gk):
    """The reference's weight_from_q8 (kernels/w8a8.py:274-286) restated: gk == 32 keeps the file's values; otherwise
    the dequantized weights are quantized again per group of gk."""
    N, K = q.shape
    if gk == 32:
        return q.contiguous(), d16.float().contiguous()
    wf = (q.view(N, K // 32, 32).float() * d16.float()[..., None]).view(N, K)
    g = wf.view(N, K // gk, gk)
    s = g.abs().amax(-1).clamp_min(1e-10) / 127.0
    return torch.round(g / s[..., None]).clamp(-127, 127).to(torch.int8).view(N, K).contiguous(), s.contiguous()


def quant_groups(x, gk):
    """Per (row, group) symmetric int8 of fp32 x with IEEE division (the activation quant contract)."""
    M, K = x.shape
    g = x.float().view(M, K // gk, gk)
    s = (g.abs().amax(-1).clamp_min(1e-10) / 127.0)
    q = torch.round(g / s[..., None]).to(torch.int8).view(M, K)   # torch.round: half to even, as rint
    return q.contiguous(), s.contiguous()


def gemm_inputs(name):
    M, N, K, live, gk, epis = GEMM_CASES[name]
    gk = gk or K
    seed = 1000 + sum(ord(c) for c in name)
    wq, wd = q8_0(torch.randn(N, K, generator=_gen(seed)) * 0.02)
    w, w_s = regroup(wq, wd, gk)
    a, a_s = quant_groups(activations(M, K, seed + 1).float(), gk)
    base = torch.randn(M, N, generator=_gen(seed + 2))
    return dict(M=M, N=N, K=K, live=live, gk=gk, epis=epis, a=a, a_s=a_s, w=w, w_s=w_s, base=base)


def swiglu_epi_inputs(name):
    M, FF, K, live, BN = SWIGLU_EPI_CASES[name]
    seed = 2000 + sum(ord(c) for c in name)
    gq, gd = q8_0(torch.randn(FF, K, generator=_gen(seed)) * 0.05)
    uq, ud = q8_0(torch.randn(FF, K, generator=_gen(seed + 1)) * 0.05)
    gate, gs = regroup(gq, gd, K)
    up, us = regroup(uq, ud, K)
    a, a_s = quant_groups(activations(M, K, seed + 2).float(), K)
    return dict(M=M, FF=FF, K=K, live=live, BN=BN, a=a, a_s=a_s, gate=gate, gate_s=gs, up=up, up_s=us)


def rows_inputs(name):
    T, K, live, with_inv = ROWS_CASES[name]
    seed = 3000 + sum(ord(c) for c in name)
    return dict(T=T, K=K, live=live, x=activations(T, K, seed), inv=inv_factors(K, seed + 1) if with_inv else None)


def swiglu_inputs(name):
    T, FF, live, with_inv = SWIGLU_CASES[name]
    seed = 4000 + sum(ord(c) for c in name)
    gu = (torch.randn(T, 2 * FF, generator=_gen(seed)) * 1.5).to(torch.bfloat16)
    return dict(T=T, FF=FF, live=live, gu=gu, inv=inv_factors(FF, seed + 1) if with_inv else None)


def norm_inputs(name):
    T, HID, live, n_parts, gather = NORM_CASES[name]
    seed = 5000 + sum(ord(c) for c in name)
    g = _gen(seed)
    R = 2 * T if gather else T
    h = activations(R, HID, seed + 1, torch.float32)
    w = 1.0 + 0.1 * torch.randn(HID, generator=g)
    rows = torch.randperm(R, generator=g)[:T].to(torch.int32) if gather else None
    parts = psa = psw = None
    if n_parts:
        parts = torch.randint(-(1 << 22), 1 << 22, (n_parts, T, HID), generator=g, dtype=torch.int32)
        psa = torch.rand(T, generator=g) * 1e-2
        psw = torch.rand(HID, generator=g) * 1e-3
    return dict(T=T, HID=HID, live=live, h=h, w=w, rows=rows, parts=parts, psa=psa, psw=psw)


def fold_inputs():
    rows, HID, live, S = FOLD_CASE
    g = _gen(6000)
    return dict(rows=rows, HID=HID, live=live, S=S, h=torch.randn(rows, HID, generator=g),
                parts=torch.randint(-(1 << 24), 1 << 24, (S, rows, HID), generator=g, dtype=torch.int32),
                a_s=torch.rand(rows, generator=g) * 1e-2, w_s=torch.rand(HID, generator=g) * 1e-3)


def groups_inputs():
    M, K, gk = GROUPS_CASE
    return dict(M=M, K=K, gk=gk, x=activations(M, K, 7000))


def gated_inputs():
    T, HV, D, live = GATED_CASE
    g = _gen(8000)
    P = 2 * HV * D + 64
    return dict(T=T, HV=HV, D=D, live=live, P=P, z_off=HV * D + 64, o=torch.randn(T, HV * D, generator=g),
                proj=torch.randn(T, P, generator=g).to(torch.bfloat16), w=1.0 + 0.1 * torch.randn(D, generator=g),
                inv=inv_factors(HV * D, 8001))


def head_inputs():
    B, HID, N, live = HEAD_CASE
    g = _gen(9000)
    wq, wd = q8_0(torch.randn(N, HID, generator=g) * 0.02)
    return dict(B=B, HID=HID, N=N, live=live, h=activations(B, HID, 9001, torch.float32),
                w=1.0 + 0.1 * torch.randn(HID, generator=g), wq=wq, wd=wd)


def mxfp4_inputs():
    M, N, K = MXFP4_CASE
    g = _gen(9500)
    return dict(M=M, N=N, K=K, x=activations(M, K, 9501), w=torch.randn(N, K, generator=g) * 0.02,
                base=torch.randn(M, N, generator=g))


def bits(t):
    """torch bf16 -> numpy uint16 bit patterns."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
