"""Seeded synthetic tensors in the on-disk formats of the path: stand-ins for GGUF model tensors and engine
activations (which no benchmark box holds).  Distributions: weights N(0, 0.02^2); activations N(0, 1) with 8 seeded
outlier channels scaled x20, cast to bf16.  Everything is generated on the CPU from torch.Generator seeds, so the CPU
oracle and the GPU see identical bytes.

Encoders (any valid block is a valid input; parity is bytes -> output):
  q8_0(w)   ggml's rule: d = max|w| / 127 (fp32), q = round(w / d), d stored as fp16.
  q4_k(w)   per 32 values a min m >= 0 and a range, 6-bit scale / min codes against fp16 d / dmin per 256 values,
            q = clamp(round((w + dmin * m) / (d * sc)), 0, 15), packed into ggml's 144-byte block.
  q6_k(w)   per 16 values an int8 scale against fp16 d per 256, q = clamp(round(w / (d * sc)), -32, 31) + 32, packed
            into ggml's 210-byte block.
"""
import torch

from . import gguf_weights as GW

TENSORS = {"qkv": (0, 7168, 5120), "o": (1, 5120, 5120), "gate_up": (2, 34816, 5120), "down": (3, 5120, 17408)}


def seed_w(cfg, tensor_index):
    return 10_000 * cfg + tensor_index


def seed_x(cfg, tensor_index, M):
    return 1_000_000 + 10_000 * cfg + 100 * tensor_index + max(M - 1, 0).bit_length()


def weights(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, k, generator=g) * 0.02


def activations(m, k, seed, outliers=8):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    idx = torch.randint(0, k, (outliers,), generator=g)
    x[:, idx] *= 20.0
    return x.to(torch.bfloat16)


def q8_0(w):
    """fp32 [n, k] -> gguf_weights.Q8 by ggml's quantize_row_q8_0 rule."""
    n, k = w.shape
    b = w.reshape(n, k // 32, 32).to(torch.float32)
    d = b.abs().amax(-1) / 127.0
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(b * inv[..., None]).clamp(-127, 127).to(torch.int8).reshape(n, k)
    return GW.Q8(q, d.to(torch.float16))


def _pack_scale_min(sc, mn):
    """Eight 6-bit scales and mins [n, 8] (integers) -> the 12 packed bytes [n, 12] (inverse of scale_min_k4)."""
    sc, mn = sc.to(torch.int32), mn.to(torch.int32)
    b = torch.zeros(sc.shape[0], 12, dtype=torch.int32)
    b[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    b[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    b[:, 8:12] = (sc[:, 4:8] & 15) | ((mn[:, 4:8] & 15) << 4)
    return b.to(torch.uint8)


def q4_k(w):
    """fp32 [n, k] -> gguf_weights.KQuant of type Q4_K."""
    n, k = w.shape
    x = w.reshape(-1, 8, 32).to(torch.float32)                        # [blocks, sub-block, 32]
    lo = x.amin(-1).clamp_max(0.0)
    hi = x.amax(-1)
    scale = (hi - lo) / 15.0                                          # per sub-block step and offset (>= 0)
    mins = -lo
    d = (scale.amax(-1) / 63.0).to(torch.float16)
    dmin = (mins.amax(-1) / 63.0).to(torch.float16)
    df, dmf = d.float(), dmin.float()
    sc = torch.where(df[:, None] > 0, torch.round(scale / df[:, None].clamp_min(1e-30)), torch.zeros_like(scale))
    mn = torch.where(dmf[:, None] > 0, torch.round(mins / dmf[:, None].clamp_min(1e-30)), torch.zeros_like(mins))
    sc, mn = sc.clamp(0, 63), mn.clamp(0, 63)
    step = df[:, None] * sc
    q = torch.where(step[..., None] > 0, torch.round((x + (dmf[:, None] * mn)[..., None]) / step[..., None].clamp_min(1e-30)),
                    torch.zeros_like(x)).clamp(0, 15).to(torch.int32)
    q = q.reshape(-1, 4, 2, 32)                                       # pairs of sub-blocks share 32 bytes
    qb = (q[:, :, 0] | (q[:, :, 1] << 4)).to(torch.uint8).reshape(-1, 128)
    raw = torch.cat([d.view(torch.uint8).reshape(-1, 2), dmin.view(torch.uint8).reshape(-1, 2),
                     _pack_scale_min(sc, mn), qb], 1)
    return GW.KQuant(raw.reshape(n, k // 256, 144).contiguous(), GW.GGML_Q4_K, k)


def q6_k(w):
    """fp32 [n, k] -> gguf_weights.KQuant of type Q6_K."""
    n, k = w.shape
    x = w.reshape(-1, 16, 16).to(torch.float32)                       # [blocks, sub-block of 16, 16]
    amax = x.abs().amax(-1)
    sub = amax / 31.0                                                 # ideal step of each sub-block
    d = (sub.amax(-1) / 127.0).to(torch.float16)
    df = d.float()
    sc = torch.where(df[:, None] > 0, torch.round(sub / df[:, None].clamp_min(1e-30)), torch.zeros_like(sub)).clamp(0, 127)
    step = df[:, None] * sc
    q = torch.where(step[..., None] > 0, torch.round(x / step[..., None].clamp_min(1e-30)), torch.zeros_like(x))
    u = (q.clamp(-32, 31) + 32).to(torch.int32).reshape(-1, 2, 4, 32)  # [block, half, quarter, 32]
    ql = torch.empty(u.shape[0], 2, 64, dtype=torch.int32)
    ql[:, :, :32] = (u[:, :, 0] & 15) | ((u[:, :, 2] & 15) << 4)
    ql[:, :, 32:] = (u[:, :, 1] & 15) | ((u[:, :, 3] & 15) << 4)
    qh = (u[:, :, 0] >> 4) | ((u[:, :, 1] >> 4) << 2) | ((u[:, :, 2] >> 4) << 4) | ((u[:, :, 3] >> 4) << 6)
    raw = torch.cat([ql.reshape(-1, 128).to(torch.uint8), qh.reshape(-1, 64).to(torch.uint8),
                     sc.to(torch.int8).view(torch.uint8).reshape(-1, 16), d.view(torch.uint8).reshape(-1, 2)], 1)
    return GW.KQuant(raw.reshape(n, k // 256, 210).contiguous(), GW.GGML_Q6_K, k)
