"""Generates the golden fixtures of tests/golden/*.npz by running the reference's own CPU-runnable code.

Run where the reference checkout is mounted (not on the GPU box):

    python tests/golden/make_golden.py [/path/to/reference]

Inputs are small seeded tensors; k-quant inputs are blocks made by prism_b200.synth's encoders (any valid block is a
valid input).  What is recorded, per file:
  w8a8.npz   kernels/w8a8.py weight_from_q8 (gk 32 / 64 / K, with and without smoothing), interleave_gate_up;
             gguf_weights.Q8.dequant
  kquant.npz gguf_weights.KQuant.dequant (Q4_K, Q5_K-free, Q6_K) and as_q8, _scale_min_k4
  w4a8.npz   kernels/w4a8.py repack (both kinds), quantize_ref, group_sums, gemm_ref, and fma32 samples
  mxfp4.npz  kernels/mxfp4.py pack ("max", "mse"), dequant_packed, the exact-grid vector of tests/test_mxfp4.py:34-38,
             and quantize_act run through Triton's CPU interpreter (TRITON_INTERPRET=1: the kernel's own code with
             numpy's log2 / exp2)
  tp.npz     tp.shard_index / shard_config for a 27B-like head layout at 2 and 4 ranks
  sims.npz   tests/quant_sim.py int8_rows / int8_groups(32) / mxfp4 fake-quantizers (the timed CPU baseline's steps)
"""
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py <path to a StartLux-Prism checkout>")
REF = sys.argv[1]
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "tests"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

from prism_b200 import synth  # noqa: E402
from startlux_prism import gguf_weights as RGW  # noqa: E402
from startlux_prism import tp as RTP  # noqa: E402
from startlux_prism.gguf import GGML_Q4_K, GGML_Q6_K  # noqa: E402
from startlux_prism.kernels import mxfp4 as RMX  # noqa: E402
from startlux_prism.kernels import w4a8 as RW4  # noqa: E402
from startlux_prism.kernels import w8a8 as RW8  # noqa: E402

import quant_sim as RSIM  # noqa: E402


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.view(torch.int16).numpy().view(np.uint16) if v.dtype == torch.bfloat16 else v.numpy()
        out[k] = np.ascontiguousarray(v)
    np.savez_compressed(os.path.join(HERE, name), **out)
    print(name, {k: (v.shape, str(v.dtype)) for k, v in out.items()})


def main():
    g = torch.Generator().manual_seed(1234)
    # ---- w8a8
    q8 = synth.q8_0(synth.weights(16, 256, 11))
    rq8 = RGW.Q8(q8.qs, q8.d)
    smooth = torch.exp(torch.randn(256, generator=g) * 0.3)
    arrs = dict(qs=q8.qs, d=q8.d, smooth=smooth, dequant=rq8.dequant(torch.float32))
    for gk, sm in ((32, None), (64, None), (256, None), (256, smooth), (32, smooth)):
        q, s = RW8.weight_from_q8(rq8, gk, sm)
        tag = f"gk{gk}{'s' if sm is not None else ''}"
        arrs[f"q_{tag}"], arrs[f"s_{tag}"] = q, s
    gate, up = torch.randint(-127, 128, (64, 32), generator=g, dtype=torch.int8), torch.randint(
        -127, 128, (64, 32), generator=g, dtype=torch.int8)
    arrs.update(gate=gate, up=up, gu16=RW8.interleave_gate_up(gate, up, 16))
    save("w8a8.npz", **arrs)
    # ---- k-quants
    w = synth.weights(24, 512, 21)
    k4, k6 = synth.q4_k(w), synth.q6_k(w)
    r4, r6 = RGW.KQuant(k4.raw, GGML_Q4_K, 512), RGW.KQuant(k6.raw, GGML_Q6_K, 512)
    a4, a6 = r4.as_q8(), r6.as_q8()
    sc, mn = RGW._scale_min_k4(k4.raw.reshape(-1, 144)[:, 4:16].to(torch.int32))
    save("kquant.npz", w=w, raw4=k4.raw, raw6=k6.raw, deq4=r4.dequant(torch.float32), deq6=r6.dequant(torch.float32),
         q8_4_qs=a4.qs, q8_4_d=a4.d, q8_6_qs=a6.qs, q8_6_d=a6.d, sc=sc, mn=mn)
    # ---- w4a8
    x = synth.activations(5, 512, 31, outliers=8).float()
    xq, a, xs = RW4.quantize_ref(x)
    arrs = dict(x=x, xq=xq, a=a, xs=xs, sums=RW4.group_sums(xs))
    for tag, r in (("4", r4), ("6", r6)):
        w4 = RW4.repack(r)
        arrs[f"q{tag}"], arrs[f"sc{tag}"], arrs[f"d{tag}"] = w4.q, w4.sc, w4.d
        if w4.mn is not None:
            arrs[f"mn{tag}"], arrs[f"dm{tag}"] = w4.mn, w4.dm
        arrs[f"y{tag}"] = RW4.gemm_ref(xq, a, xs, w4)
    fa, fb, fc = (torch.randn(4096, generator=g) * s for s in (1.0, 3.0, 2.0))
    arrs.update(fa=fa, fb=fb, fc=fc, fma=RW4.fma32(fa, fb, fc))
    save("w4a8.npz", **arrs)
    # ---- mxfp4
    wm = synth.weights(8, 256, 41)
    arrs = dict(w=wm)
    for mode in ("max", "mse"):
        m = RMX.pack(wm, mode)
        arrs[f"q_{mode}"], arrs[f"s_{mode}"], arrs[f"deq_{mode}"] = m.q, m.s, RMX.dequant_packed(m.q, m.s)
    grid = torch.tensor([[0.0, 0.5, -0.5, 1.0, -1.0, 1.5, 2.0, 3.0, 4.0, 6.0] * 3 + [0.0, 0.5]])
    mg = RMX.pack(grid)
    arrs.update(grid=grid, grid_q=mg.q, grid_s=mg.s, grid_deq=RMX.dequant_packed(mg.q, mg.s))
    xa = synth.activations(6, 512, 51)
    for tag, xin in (("bf16", xa), ("f32", xa.float() * 0.37)):
        q = torch.zeros(6, 256, dtype=torch.uint8)
        s = torch.zeros(6, 16, dtype=torch.uint8)
        RMX.quantize_act(xin, q, s)
        arrs[f"act_{tag}"], arrs[f"act_q_{tag}"], arrs[f"act_s_{tag}"] = xin, q, s
    inv = torch.exp(torch.randn(512, generator=g) * 0.1)
    q = torch.zeros(6, 256, dtype=torch.uint8)
    s = torch.zeros(6, 16, dtype=torch.uint8)
    RMX.quantize_act_scaled(xa, inv, q, s)
    arrs.update(act_inv=inv, act_q_scaled=q, act_s_scaled=s)
    save("mxfp4.npz", **arrs)
    # ---- tp
    cfg = types.SimpleNamespace(n_head=20, n_kv_head=4, head_dim=128, k_heads=16, v_heads=48, gdn_dim=128, ffn=17408)
    arrs = {}
    for n in (2, 4):
        for r in range(n):
            for k, v in RTP.shard_index(cfg, n, r).items():
                arrs[f"n{n}_r{r}_{k}"] = v
    save("tp.npz", **arrs)
    # ---- the CPU emulation's fake-quantizers
    xs_ = synth.activations(4, 256, 61).float()
    save("sims.npz", x=xs_, int8_rows=RSIM.int8_rows(xs_), int8_g32=RSIM.int8_groups(32)(xs_), mxfp4=RSIM.mxfp4(xs_))


if __name__ == "__main__":
    main()
