"""MXFP4 projections: the operator API of the reference's kernels/mxfp4.py over the sm_100a library.

    MX4(q, s, n, k, cs)                 packed weights: codes uint8 [n, k/2], scales uint8 [n, k/32]  (mxfp4.py:25-37)
    pack(w, mode)                       fp32 / bf16 matrix -> MX4 ("max" or "mse" scale choice)          (mxfp4.py:57-86)
    dequant_packed(q, s)                fp32 values of a packed operand                                  (mxfp4.py:89-101)
    quantize_act(x, q, s)               activation rows -> the same format, on the GPU                   (mxfp4.py:182-185)
    quantize_act_scaled(x, inv, q, s)   with a per-column pre-scale                                      (mxfp4.py:174-179)
    prepare(w)                          MX4 with its scales in the tensor core's tiled order (cs)        (mxfp4.py:214-224)
    gemm(a_q, a_s, w, out, n_rows, epi) out = deq(a) deq(w)^T, fp32 accumulate                           (mxfp4.py:292-317)
    gemv(a_q, a_s, w, out, n_rows, epi) the same for one to four rows on the CUDA cores (no counterpart)

Values: e2m1 grid 0, .5, 1, 1.5, 2, 3, 4, 6 with sign bit 8, nearest with strict thresholds; block scale
2^ceil(log2(amax / 6)) clipped to 2^+-127, stored as e + 127; byte = code[2i] | code[2i + 1] << 4.
"""
from __future__ import annotations

from typing import NamedTuple

import numpy as np
import torch

from . import _lib

QK = 32
_LUT = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
_ACT_SF = {}


class MX4(NamedTuple):
    q: torch.Tensor
    s: torch.Tensor
    n: int
    k: int
    cs: torch.Tensor | None = None      # scales in the tensor core's tiled order (prepare)

    @property
    def shape(self):
        return (self.n, self.k)

    def rows(self, r0, r1):
        return MX4(self.q[r0:r1], self.s[r0:r1], r1 - r0, self.k)


def _codes(x):
    """x / scale (numpy fp32) -> 4-bit e2m1 codes: nearest magnitude, midpoints round down, sign bit unless zero."""
    a = np.abs(x)
    c = np.zeros(a.shape, np.uint8)
    for code, bound in enumerate((0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0), start=1):
        c[a > bound] = code
    c[(x < 0) & (c != 0)] |= 8
    return c


def pack(w: torch.Tensor, mode: str = "max") -> MX4:
    """A [n, k] matrix -> MX4 on the CPU (load time).  "max": the smallest power of two that keeps the block's maximum
    within the grid; "mse": that one or half of it, whichever has the smaller squared error in the block."""
    x = w.detach().to(torch.float32).cpu().numpy()
    n, k = x.shape
    if k % QK:
        raise ValueError(f"k = {k} is not a multiple of {QK}")
    b = x.reshape(n, k // QK, QK)
    amax = np.abs(b).max(axis=2)
    with np.errstate(divide="ignore"):
        e = np.clip(np.ceil(np.log2(np.maximum(amax, 1e-30) / 6.0)), -127, 127)
    if mode == "mse":
        e1 = np.clip(e - 1, -127, 127)
        err = []
        for ee in (e, e1):
            sc = np.exp2(ee).astype(np.float32)[..., None]
            err.append(((_LUT[_codes(b / sc)] * sc - b) ** 2).sum(axis=2))
        e = np.where(err[1] < err[0], e1, e)
    elif mode != "max":
        raise ValueError(f"mode {mode!r}")
    code = _codes(b / np.exp2(e).astype(np.float32)[..., None]).reshape(n, k)
    q = (code[:, 0::2] | (code[:, 1::2] << 4)).astype(np.uint8)
    s = (e.astype(np.int16) + 127).astype(np.uint8).reshape(n, k // QK)
    return MX4(torch.from_numpy(q).contiguous(), torch.from_numpy(s).contiguous(), n, k)


def dequant_packed(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """fp32 [n, k] of packed codes and scales (CPU; tests and load-time checks)."""
    qn = q.cpu().numpy()
    n, k2 = qn.shape
    out = np.empty((n, 2 * k2), np.float32)
    out[:, 0::2], out[:, 1::2] = _LUT[qn & 15], _LUT[qn >> 4]
    sc = np.exp2(s.cpu().numpy().astype(np.int16) - 127).astype(np.float32)
    return torch.from_numpy((out.reshape(n, -1, QK) * sc[..., None]).reshape(n, 2 * k2))


def _quant(x, inv, q, s):
    n, k = x.shape
    _lib.need_cuda(x, q, s, inv)
    if x.dtype not in (torch.bfloat16, torch.float32) or not x.is_contiguous():
        raise RuntimeError("quantize_act: x must be contiguous bf16 or fp32")
    if q.dtype != torch.uint8 or s.dtype != torch.uint8 or q.shape[1] != k // 2 or s.shape[1] != k // QK \
            or not q.is_contiguous() or not s.is_contiguous():
        raise RuntimeError("quantize_act: q uint8 [n, k/2], s uint8 [n, k/32], contiguous")
    rc = _lib.lib().pb_mxfp4_quant(_lib.ptr(x), int(x.dtype == torch.float32), _lib.ptr(inv), _lib.ptr(q),
                                   _lib.ptr(s), n, k, _lib.stream())
    _lib.check(rc, f"mxfp4 quantize_act n={n} k={k}")


def quantize_act(x: torch.Tensor, q: torch.Tensor, s: torch.Tensor) -> None:
    """x [n, k] bf16 / fp32 -> q uint8 [n, k/2], s uint8 [n, k/32] (the caller's buffers)."""
    _quant(x, None, q, s)


def quantize_act_scaled(x: torch.Tensor, inv: torch.Tensor, q: torch.Tensor, s: torch.Tensor) -> None:
    """quantize_act of x * inv (inv fp32 [k]: an already smoothed input)."""
    _quant(x, inv, q, s)


def _tile_scales(s, rows, k):
    nbytes = _lib.lib().pb_mxfp4_sf_bytes(rows, k)
    if nbytes == 0:
        raise RuntimeError(f"mxfp4: k = {k} must be a multiple of 128")
    dst = torch.empty(nbytes, dtype=torch.uint8, device=s.device)
    rc = _lib.lib().pb_mxfp4_prepare_sf(_lib.ptr(s), _lib.ptr(dst), rows, k, _lib.stream())
    _lib.check(rc, "mxfp4 prepare_sf")
    return dst


def prepare(w: MX4) -> MX4:
    """MX4 (on the GPU) with its scales also in the tensor core's tiled order; call once at load."""
    if w.cs is not None:
        return w
    _lib.need_cuda(w.q, w.s)
    return MX4(w.q.contiguous(), w.s.contiguous(), w.n, w.k, _tile_scales(w.s.contiguous(), w.n, w.k))


cutlass_prepare = prepare       # the reference's name for the same step (kernels/mxfp4.py:214)


def _sm_count():
    from .w8a8 import SM_COUNT
    return SM_COUNT


def gemv(a_q, a_s, w: MX4, out, n_rows, epi=0, out_stride=None):
    """gemm for one to four rows on the CUDA cores: exact integer products per 32-input block, one fp32 multiply-add
    per block (mxfp4_gemv_kernel).  Takes the plain scale bytes (w.s, a_s), not the tiled order; differs from gemm
    only in the order of the fp32 additions."""
    M, K, N = int(n_rows), w.k, w.n
    _lib.need_cuda(a_q, a_s, w.q, w.s, out)
    want = torch.bfloat16 if epi == 0 else torch.float32
    if out.dtype != want or out.stride(-1) != 1:
        raise RuntimeError(f"mxfp4.gemv: out must be {want} with unit column stride")
    if not a_q.is_contiguous() or not a_s.is_contiguous() or a_q.shape[1] != K // 2 or not w.s.is_contiguous():
        raise RuntimeError("mxfp4.gemv: a_q [rows, k/2], a_s [rows, k/32] and w.s must be contiguous")
    ldo = out.stride(0) if out_stride is None else out_stride
    rc = _lib.lib().pb_mxfp4_gemv(_lib.ptr(a_q), _lib.ptr(a_s), _lib.ptr(w.q), _lib.ptr(w.s), _lib.ptr(out), ldo, M, N, K,
                                  epi, _lib.stream())
    _lib.check(rc, f"mxfp4 gemv M={M} N={N} K={K} epi={epi}")


def pick_split(M, N, K):
    """K slices per 128 x 128 tile: only where one row tile's tiles leave most SMs idle (decode shapes against the
    5120-row projections); every slice keeps at least 4 K blocks of 256."""
    from .w8a8 import SM_COUNT
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    if M > 128 or tiles * 2 > SM_COUNT:
        return 1
    return max(1, min(SM_COUNT // tiles, (K // 256) // 4, 8))


def gemm(a_q, a_s, w: MX4, out, n_rows, epi=0, out_stride=None, split=None):
    """a_q uint8 [>= n_rows, k/2], a_s uint8 [>= n_rows, k/32]; w MX4 [N, k] (prepare()d, or prepared here on every
    call).  epi 0 writes bf16 into out, epi 1 adds into the fp32 residual out; out's row stride is honoured.
    split: K slices per tile; None or 1: one accumulator over all of K, so a row's bits do not depend on the batch it
    came in (the reference's batch invariance); "auto": one row against a matrix of few rows on the CUDA cores (gemv), otherwise
    pick_split (decode shapes against few-row matrices run several times faster); the slices' fp32 sums are added in slice order: deterministic, and within fp32 rounding of the
    unsplit sum."""
    M, K, N = int(n_rows), w.k, w.n
    _lib.need_cuda(a_q, a_s, w.q, out)
    if w.cs is None:
        w = prepare(w)
    want = torch.bfloat16 if epi == 0 else torch.float32
    if out.dtype != want or out.stride(-1) != 1:
        raise RuntimeError(f"mxfp4.gemm: out must be {want} with unit column stride")
    if not a_q.is_contiguous() or not a_s.is_contiguous() or a_q.shape[1] != K // 2:
        raise RuntimeError("mxfp4.gemm: a_q [rows, k/2] and a_s [rows, k/32] must be contiguous")
    if split == "auto" and M == 1 and K % 256 == 0 and (N + 7) // 8 < 8 * _sm_count():
        # one row against a matrix of few rows: the CUDA-core kernel (measured: level with the tensor-core kernel on a
        # 34816-row matrix and behind it from two rows, where its decode arithmetic is the bound)
        return gemv(a_q, a_s, w, out, M, epi, out_stride)
    key = (a_q.shape[0], K, a_q.device.index)
    need = _lib.lib().pb_mxfp4_sf_bytes(a_q.shape[0], K)
    sfa = _ACT_SF.get(key)
    if sfa is None or sfa.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("mxfp4.gemm: run this shape once eagerly before graph capture (scale buffer)")
        sfa = _ACT_SF[key] = torch.zeros(need, dtype=torch.uint8, device=a_q.device)
    L = _lib.lib()
    _lib.check(L.pb_mxfp4_prepare_sf(_lib.ptr(a_s), _lib.ptr(sfa), a_q.shape[0], K, _lib.stream()), "mxfp4 prepare_sf")
    ldo = out.stride(0) if out_stride is None else out_stride
    split = 1 if split is None else pick_split(M, N, K) if split == "auto" else max(1, int(split))
    ws = counters = None
    if split > 1:
        from . import w8a8 as KW
        ws, counters = KW._workspace(a_q.device)
        if L.pb_mxfp4_workspace_bytes(M, N, split) > ws.numel() or L.pb_mxfp4_counters(M, N) > counters.numel():
            split, ws, counters = 1, None, None
    rc = L.pb_mxfp4_gemm_split(_lib.ptr(a_q), _lib.ptr(sfa), _lib.ptr(w.q), _lib.ptr(w.cs), _lib.ptr(out), ldo, M, N, K,
                               epi, split, _lib.ptr(ws), 0 if ws is None else ws.numel(), _lib.ptr(counters),
                               0 if counters is None else counters.numel(), _lib.stream())
    _lib.check(rc, f"mxfp4 gemm M={M} N={N} K={K} epi={epi}")
