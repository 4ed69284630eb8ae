"""The decode step's vocabulary head on Q8_0 weights: the reference's kernels/decode.py head_quant / head_q8
(:113-160, :351-364) over the sm_100a library.

    head_quant(h, norm, q, s, n, B, eps)       final RMSNorm of the residual rows, int8 per 32 inputs
    head_q8(a, a_s, w, w_s, out, n, B)         logits fp32 [B, N]: over the 32-input groups, in order,
                                               acc = fma(float(a_g . w_g) * a_s[g], w_s[g], acc)
    head_scales(w_s)                           the file's group-major fp16 scales [K/32, N] -> fp32 [N, K/32] (load time)

The GEMM is the per-32-group few-rows W8A8 kernel (w8a8.gemm, gk = 32) with a plain fp32 store.  The reference's
Triton expression `acc += (ai * sa) * sw` carries no explicit roundings and its compiler fuses the second multiply
with the add; this kernel computes the same - one rounded product, then a fused multiply-add, groups in ascending
order - and equals the reference kernel's recorded logits bit for bit (tests/golden/gpu_ref.npz).
"""
from __future__ import annotations

import torch

from . import _lib, w8a8

HEAD_G = 32                         # Q8_0 block: the output head's weights as stored

_SCALES = {}


def head_quant(h, norm, q, s, n, B, eps):
    """h fp32 [>= B, HID], norm fp32 [HID] -> q int8 [>= B, HID], s fp32 [>= B, HID / 32]."""
    HID = h.shape[1]
    _lib.need_cuda(h, norm, q, s, n)
    if h.dtype != torch.float32 or not h.is_contiguous() or q.shape[1] != HID or not q.is_contiguous() \
            or s.shape[1] != HID // HEAD_G or not s.is_contiguous():
        raise RuntimeError("head_quant: h fp32 [B, HID], q int8 [B, HID], s fp32 [B, HID / 32], contiguous")
    rc = _lib.lib().pb_head_quant(_lib.ptr(h), _lib.ptr(norm), _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), B, HID, float(eps),
                                  _lib.stream())
    _lib.check(rc, f"head_quant B={B} HID={HID}")


def head_scales(w_s):
    """Group-major scales [K/32, N] (fp16 as the file stores them, or fp32) -> fp32 [N, K/32], what the kernel reads.
    Done once per tensor (cached by its storage)."""
    key = (w_s.data_ptr(), tuple(w_s.shape), w_s.dtype)
    t = _SCALES.get(key)
    if t is None:
        t = _SCALES[key] = w_s.float().t().contiguous()
    return t


def head_q8(a, a_s, w, w_s, out, n, B, bn=64, gpi=4, warps=4, stages=3):
    """a int8 [B, K], a_s fp32 [B, K/32], w int8 [N, K], w_s [K/32, N] (fp16 / fp32, group-major) or the result of
    head_scales -> out fp32 [B, N].  bn, gpi, warps, stages: accepted for signature parity (one kernel shape)."""
    N, K = w.shape
    if w_s.shape == (K // HEAD_G, N) and (N != K // HEAD_G or w_s.dtype != torch.float32):
        w_s = head_scales(w_s)
    if out.dtype != torch.float32:
        raise RuntimeError("head_q8: out must be fp32 [B, N]")
    w8a8.gemm(a[:B], a_s[:B], w, w_s, out[:B], n, HEAD_G, epi=w8a8.EPI_F32)
