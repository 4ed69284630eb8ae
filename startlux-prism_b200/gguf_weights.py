"""GGUF weight containers on the quantized linear-layer path: Q8_0 matrices (Q8) and llama.cpp k-quant matrices
(KQuant: Q4_K, Q5_K, Q6_K) with their exact dequantization.  Counterpart of the reference's gguf_weights.py:30-133
(Q8, _scale_min_k4, _dq_q4_k, _dq_q5_k, _dq_q6_k, KQuant.dequant, KQuant.as_q8); the model-level loader (Config,
Layer, load) is engine code and not part of this package.

Block formats (ggml):
  Q8_0  34 bytes per 32 values: fp16 d, 32 int8 q; w = d * q.
  Q4_K  144 bytes per 256: fp16 d, fp16 dmin, 12 bytes holding eight 6-bit scales and eight 6-bit mins, 128 bytes of
        nibbles (each 32 bytes hold two 32-value sub-blocks: low nibbles first); w = d * sc * q - dmin * m.
  Q5_K  176 bytes: as Q4_K plus 32 bytes with the fifth bit of every value.
  Q6_K  210 bytes per 256: 128 bytes of low nibbles, 64 bytes of 2-bit tops, 16 int8 scales (one per 16 values),
        fp16 d; w = d * sc * (q - 32).
"""
from __future__ import annotations

import dataclasses

import torch

GGML_Q8_0, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K = 8, 12, 13, 14
BLOCK_BYTES = {GGML_Q8_0: 34, GGML_Q4_K: 144, GGML_Q5_K: 176, GGML_Q6_K: 210}
QK = 32
QK_K = 256


@dataclasses.dataclass
class Q8:
    """A Q8_0 matrix [n, k]: qs int8 [n, k], d fp16 [n, k / 32]."""
    qs: torch.Tensor
    d: torch.Tensor

    @property
    def shape(self):
        return tuple(self.qs.shape)

    def to(self, device):
        return Q8(self.qs.to(device), self.d.to(device))

    def dequant(self, dtype=torch.float32, rows=None):
        qs, d = (self.qs, self.d) if rows is None else (self.qs[rows], self.d[rows])
        blocks = qs.reshape(*qs.shape[:-1], qs.shape[-1] // QK, QK).to(torch.float32)
        return (blocks * d.to(torch.float32)[..., None]).reshape(qs.shape).to(dtype)

    @staticmethod
    def from_blocks(raw, n, k):
        """raw uint8 [n * k / 32 * 34] (the file's bytes) -> Q8."""
        b = raw.reshape(n, k // QK, 34)
        d = b[..., :2].contiguous().view(torch.float16).reshape(n, k // QK)
        qs = b[..., 2:].contiguous().view(torch.int8).reshape(n, k)
        return Q8(qs, d)


def _half(b):
    return b.contiguous().view(torch.float16).to(torch.float32)


def scale_min_k4(s):
    """The eight 6-bit scales and eight 6-bit mins packed in 12 bytes of a Q4_K / Q5_K super-block: s integer
    [n, 12] -> (sc [n, 8], mn [n, 8]) as integers.  Bytes 0-3 / 4-7 carry the low 6 bits of scales / mins 0-3 and, in
    their top 2 bits, bits 4-5 of scales / mins 4-7, whose low nibbles sit in bytes 8-11."""
    s = s.to(torch.int32)
    lo, mid, hi = s[:, 0:4], s[:, 4:8], s[:, 8:12]
    sc = torch.cat([lo & 63, (hi & 15) | ((lo >> 6) << 4)], 1)
    mn = torch.cat([mid & 63, (hi >> 4) | ((mid >> 6) << 4)], 1)
    return sc, mn


def _nibbles_k(qbytes):
    """128 bytes of Q4_K / Q5_K quants -> integers [n, 8, 32] in input order."""
    q = qbytes.to(torch.int32).reshape(-1, 4, 32)
    return torch.stack([q & 15, q >> 4], 2).reshape(-1, 8, 32)


def q6k_values(b):
    """Q6_K blocks uint8 [n, 210] -> the 6-bit values (0..63) as integers [n, 256] in input order."""
    ql, qh = b[:, :128].to(torch.int32), b[:, 128:192].to(torch.int32)
    out = []
    for half in range(2):
        l0, l1 = ql[:, 64 * half:64 * half + 32], ql[:, 64 * half + 32:64 * half + 64]
        top = qh[:, 32 * half:32 * half + 32]
        out += [(l0 & 15) | ((top & 3) << 4), (l1 & 15) | (((top >> 2) & 3) << 4),
                (l0 >> 4) | (((top >> 4) & 3) << 4), (l1 >> 4) | (((top >> 6) & 3) << 4)]
    return torch.cat(out, 1)


def dequant_q4_k(b):
    d, dmin = _half(b[:, 0:2]), _half(b[:, 2:4])
    sc, mn = scale_min_k4(b[:, 4:16])
    q = _nibbles_k(b[:, 16:144]).to(torch.float32)
    y = (d * sc.to(torch.float32))[:, :, None] * q - (dmin * mn.to(torch.float32))[:, :, None]
    return y.reshape(-1, QK_K)


def dequant_q5_k(b):
    d, dmin = _half(b[:, 0:2]), _half(b[:, 2:4])
    sc, mn = scale_min_k4(b[:, 4:16])
    qh = b[:, 16:48].to(torch.int32)
    q = _nibbles_k(b[:, 48:176])
    fifth = torch.stack([(qh >> i) & 1 for i in range(8)], 1)
    q = (q | (fifth << 4)).to(torch.float32)
    y = (d * sc.to(torch.float32))[:, :, None] * q - (dmin * mn.to(torch.float32))[:, :, None]
    return y.reshape(-1, QK_K)


def dequant_q6_k(b):
    sc = b[:, 192:208].contiguous().view(torch.int8).to(torch.float32)
    d = _half(b[:, 208:210])
    q = q6k_values(b).to(torch.float32) - 32
    return (d * sc).repeat_interleave(16, 1) * q


_DEQUANT = {GGML_Q4_K: dequant_q4_k, GGML_Q5_K: dequant_q5_k, GGML_Q6_K: dequant_q6_k}


@dataclasses.dataclass
class KQuant:
    """A k-quant matrix [n, k] as its raw super-blocks: raw uint8 [n, k / 256, block bytes]."""
    raw: torch.Tensor
    type: int
    k: int

    @property
    def shape(self):
        return (self.raw.shape[0], self.k)

    def to(self, device):
        return KQuant(self.raw.to(device), self.type, self.k)

    def dequant(self, dtype=torch.float32, rows=None):
        raw = self.raw if rows is None else self.raw[rows]
        y = _DEQUANT[self.type](raw.reshape(-1, raw.shape[-1]))
        return y.reshape(*raw.shape[:-2], self.k).to(dtype)

    def as_q8(self, chunk=16384):
        """Q8_0 blocks of the dequantized values: d = fp16(max|w| / 127), q = round(w / d) clamped to +-127 (a zero
        block keeps q = 0)."""
        n, k = self.shape
        qs = torch.empty(n, k, dtype=torch.int8, device=self.raw.device)
        d = torch.empty(n, k // QK, dtype=torch.float16, device=self.raw.device)
        for i in range(0, n, chunk):
            wv = self.dequant(torch.float32, slice(i, i + chunk)).view(-1, k // QK, QK)
            dh = (wv.abs().amax(-1) / 127).half()
            inv = torch.where(dh > 0, 1.0 / dh.float(), torch.zeros_like(dh, dtype=torch.float32))
            qs[i:i + chunk] = torch.round(wv * inv[..., None]).clamp(-127, 127).to(torch.int8).view(-1, k)
            d[i:i + chunk] = dh
        return Q8(qs, d)
