"""The reference's CPU emulation of the W8A8 path, restated: the timed CPU baseline of the benchmark.

TEST / BENCH INFRASTRUCTURE ONLY (never imported by the product package).  The reference simulates its int8 path on
the CPU by fake-quantizing both operands onto their int8 grids and multiplying in fp32 with torch
(tests/quant_sim.py:97-107 int8_rows / int8_groups; tests/int8_sim.py:75-81 w8a8: per-token activation grid, per-row
weight grid, `xq @ wq.T`; startlux_prism/reference.py:40-41 linear).  It is a simulation, not the bit oracle: fp32
sums of int8 products are not exact beyond 2^24.  Pinned by tests/golden/sims.npz (tests/test_oracle.py).
"""
import os
import time

import torch


def int8_rows(x):
    """Fake-quantize each row onto its symmetric int8 grid (tests/quant_sim.py:97-99)."""
    sc = x.abs().amax(-1, keepdim=True).clamp_min(1e-10) / 127
    return torch.round(x / sc).clamp(-127, 127) * sc


def int8_groups(g):
    """Fake-quantize each group of g inputs onto its own int8 grid (tests/quant_sim.py:102-107)."""
    def q(x):
        b = x.reshape(*x.shape[:-1], -1, g)
        sc = b.abs().amax(-1, keepdim=True).clamp_min(1e-10) / 127
        return (torch.round(b / sc).clamp(-127, 127) * sc).reshape(x.shape)
    return q


def linear(x, w_fake):
    """tests/int8_sim.py:75-81 without smoothing: per-token fake-quantized activations times fake-quantized weights."""
    return int8_rows(x) @ w_fake.T


class LayerSet:
    """One decoder layer's linear set on the CPU, weights fake-quantized once (load time, not timed)."""
    SHAPES = {"qkv": (7168, 5120), "o": (5120, 5120), "gate_up": (34816, 5120), "down": (5120, 17408)}

    def __init__(self, seed=0, threads=None):
        torch.set_num_threads(threads or os.cpu_count())
        self.threads = torch.get_num_threads()
        g = torch.Generator().manual_seed(seed)
        self.w = {k: int8_rows(torch.randn(n, kk, generator=g) * 0.02) for k, (n, kk) in self.SHAPES.items()}
        self.ops_per_row = 2 * sum(n * k for n, k in self.SHAPES.values())

    def run(self, h):
        """h fp32 [rows, 5120] -> (seconds, ops) of one layer: q|k|v, o (+residual), gate|up, SwiGLU, down (+residual)."""
        t0 = time.perf_counter()
        qkv = linear(h, self.w["qkv"])
        h = h + linear(qkv[:, :5120], self.w["o"])
        gu = linear(h, self.w["gate_up"])
        act = torch.nn.functional.silu(gu[:, :17408]) * gu[:, 17408:]
        h = h + linear(act, self.w["down"])
        return time.perf_counter() - t0, self.ops_per_row * h.shape[0], h
