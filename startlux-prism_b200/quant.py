"""Producers of quantized projection inputs and the deferred residual add: the operator API of the reference's
kernels/quant.py over the sm_100a library.

    rows_q8(x, inv_s, q, s, n, T, mode, amax)     x bf16 [T, K] * inv_s -> int8 + per-token scale  (quant.py:481-486)
    swiglu_q8(gu, inv_s, q, s, n, T, mode, amax)  silu(gate) * up -> int8 + per-token scale         (quant.py:473-478)
    rows_g(x, q, s, xs, n, T)                     W4A8: scale per 256 inputs + split group sums     (quant.py:408-411)
    fold(h, parts, pending, n, T)                 finish a w8a8.Deferred residual add               (quant.py:448-457)

Tensor-parallel modes (quant.py:14-27): 1 also stores the row's own maximum in `amax`, 2 quantizes with
max(amax[t], own) after `amax` was max-all-reduced, 3 exchanges the maxima with the other ranks inside the launch (a
Sync from tp.Group.words(): one 64-bit word per row and rank, pass number above the float's bits, written into every
other rank's buffer over NVLink); a maximum is exact in any order, so every rank's int8 values and scales are the
single-GPU kernel's.  fold and norm_q8 take a Deferred whose `sync` (tp.Group.sync()) makes them add every rank's
int32 slots themselves, read over NVLink after a flag handshake, instead of an all-reduce between two kernels
(quant.py:29-37).  Every device-side wait is bounded (a rank that never arrives gives PrismError status 4 through
_lib.device_status, not a hang).
"""
import ctypes
from typing import NamedTuple

import torch

from . import _lib


class Sync(NamedTuple):
    """One in-kernel exchange step of a tensor-parallel group (the reference's quant.Sync, kernels/quant.py:55-65):
    `epoch` int64 [1] on the device, the pass number (the same on every rank); `flags`: every rank's 64-bit word buffer
    as mapped on this GPU, in rank order (tensors or raw device addresses); `chan`: for a flag handshake the step's
    channel, for a row-maximum exchange the first word row of the step; `others`: the other ranks' int32 slot buffers
    as mapped here (folds only); this process's rank and the group's size."""
    epoch: torch.Tensor
    flags: tuple
    chan: int
    others: tuple
    rank: int
    world: int


def _addr(t):
    return int(t) if isinstance(t, int) else t.data_ptr()


def _sync_struct(sync):
    st = _lib.SyncStruct()
    st.epoch = sync.epoch.data_ptr()
    if len(sync.flags) != sync.world or sync.world > 8:
        raise RuntimeError(f"Sync: {len(sync.flags)} buffers for {sync.world} ranks (at most 8)")
    for r, f in enumerate(sync.flags):
        st.bufs[r] = _addr(f)
    for r, o in enumerate(sync.others):
        st.others[r] = _addr(o)
    st.off, st.rank, st.world = int(sync.chan), int(sync.rank), int(sync.world)
    return st


def bump(epoch):
    """A new pass number (int64 [1], device) at the start of a tensor-parallel pass; every rank runs the same passes, so
    they count alike.  A device-side add on the current stream: graph-capturable (kernels/quant.py:78-87)."""
    epoch.add_(1)


def push(src, dsts):
    """src (contiguous, a multiple of 16 bytes) stored into each of dsts: the same block of the other ranks' buffers as
    mapped on this GPU (tp.Group.symmetric).  The receivers may read it after handshake()."""
    _lib.need_cuda(src)
    if not src.is_contiguous() or any(d.numel() * d.element_size() != src.numel() * src.element_size() for d in dsts):
        raise RuntimeError("push: contiguous blocks of one size")
    arr = (ctypes.c_void_p * max(len(dsts), 1))(*[d.data_ptr() for d in dsts])
    rc = _lib.lib().pb_push(_lib.ptr(src), arr, len(dsts), src.numel() * src.element_size(), _lib.stream())
    _lib.check(rc, f"push {src.numel() * src.element_size()} bytes to {len(dsts)} ranks")


def handshake(sync):
    """The flag handshake of `sync` (tp.Group.handshake()) as a step of its own on the stream: signals every other rank
    and waits (bounded) for all of them."""
    rc = _lib.lib().pb_handshake(ctypes.byref(_sync_struct(sync)), _lib.stream())
    _lib.check(rc, f"handshake over {sync.world} ranks")


def _mode_args(mode, amax, sync, T):
    if mode == 3:
        if sync is None:
            raise RuntimeError("mode 3 needs a Sync (tp.Group.words())")
        if sync.flags and hasattr(sync.flags[0], "numel") and sync.flags[0].numel() < (sync.chan + T) * sync.world:
            raise RuntimeError("mode 3: the word buffers are too small for this many rows (tp.Group.setup / setup_many)")
        return None
    if sync is not None:
        raise RuntimeError("a Sync goes with mode 3")
    if mode not in (0, 1, 2):
        raise ValueError(f"mode {mode}")
    if mode and (amax is None or amax.dtype != torch.float32 or amax.numel() < T):
        raise RuntimeError("modes 1 / 2 need an fp32 amax buffer of at least T elements")
    return amax if mode else None


def rows_q8(x, inv_s, q, s, n, T, mode=0, amax=None, sync=None):
    """x bf16 / fp32 [>= T, K] (rows may be strided: a column slice of a wider buffer), inv_s fp32 [K] or None ->
    q int8 [>= T, K], s fp32 [>= T]; n: device int32 live rows."""
    K = q.shape[1]
    _lib.need_cuda(x, q, s, n)
    amax = _mode_args(mode, amax, sync, T)
    if x.dtype not in (torch.bfloat16, torch.float32) or x.shape[1] != K or x.stride(1) != 1 or not q.is_contiguous():
        raise RuntimeError("rows_q8: x must be bf16 / fp32 [T, K] with unit column stride, matching q")
    if mode == 3:
        rc = _lib.lib().pb_quant_rows_exchange(_lib.ptr(x), int(x.dtype == torch.float32), x.stride(0), _lib.ptr(inv_s),
                                               _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), T, K,
                                               ctypes.byref(_sync_struct(sync)), _lib.stream())
    else:
        rc = _lib.lib().pb_quant_rows(_lib.ptr(x), int(x.dtype == torch.float32), x.stride(0), _lib.ptr(inv_s),
                                      _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), T, K, K, mode, _lib.ptr(amax), _lib.stream())
    _lib.check(rc, f"rows_q8 T={T} K={K} mode={mode}")


def swiglu_q8(gu, inv_s, q, s, n, T, mode=0, amax=None, sync=None):
    """gu bf16 [>= T, 2 FF] (gate columns then up columns) -> q int8 [>= T, FF], s fp32 [>= T]."""
    FF = q.shape[1]
    _lib.need_cuda(gu, q, s, n)
    amax = _mode_args(mode, amax, sync, T)
    if gu.dtype != torch.bfloat16 or gu.shape[1] != 2 * FF or not gu.is_contiguous() or not q.is_contiguous():
        raise RuntimeError("swiglu_q8: gu must be contiguous bf16 [T, 2 FF]")
    if mode == 3:
        rc = _lib.lib().pb_swiglu_q8_exchange(_lib.ptr(gu), _lib.ptr(inv_s), _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), T, FF,
                                              ctypes.byref(_sync_struct(sync)), _lib.stream())
    else:
        rc = _lib.lib().pb_swiglu_q8(_lib.ptr(gu), _lib.ptr(inv_s), _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), T, FF, mode,
                                     _lib.ptr(amax), _lib.stream())
    _lib.check(rc, f"swiglu_q8 T={T} FF={FF} mode={mode}")


def norm_q8(h, w_over_s, q, s, n, T, eps, rows=None, parts=None, pending=None):
    """RMSNorm + per-token int8 (the reference's norm_q8, kernels/quant.py:418-431): h fp32 [rows, HID] -> q int8
    [>= T, HID], s fp32 [>= T]; output row i reads h[rows[i]] when rows (int32, device) is given.  pending (a
    w8a8.Deferred) with parts int32 [S, rows, HID]: the residual add a split-K projection left open is finished in h
    first (and stored).  The deferred projection's activation scales may be `s` itself."""
    HID = h.shape[1]
    _lib.need_cuda(h, w_over_s, q, s, n)
    if h.dtype != torch.float32 or not h.is_contiguous() or w_over_s.dtype != torch.float32 or q.shape[1] != HID:
        raise RuntimeError("norm_q8: h fp32 [rows, HID] contiguous, w fp32 [HID], q int8 [T, HID]")
    np_ = pending.n if pending else 0
    if np_ and pending.parts is not None:
        parts = pending.parts
    if np_ and (parts is None or rows is not None or parts.dtype != torch.int32):
        raise RuntimeError("norm_q8: a pending add needs its int32 slots and no row gather")
    if np_ and getattr(pending, "sync", None) is not None:
        rc = _lib.lib().pb_norm_q8_sync(_lib.ptr(h), _lib.ptr(w_over_s), _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), T, HID,
                                        float(eps), _lib.ptr(parts), parts.stride(0), np_, _lib.ptr(pending.a_s),
                                        _lib.ptr(pending.w_s), ctypes.byref(_sync_struct(pending.sync)), _lib.stream())
        _lib.check(rc, f"norm_q8 T={T} HID={HID} parts={np_} over {pending.sync.world} ranks")
        return
    rc = _lib.lib().pb_norm_q8(_lib.ptr(h), _lib.ptr(w_over_s), _lib.ptr(q), _lib.ptr(s), _lib.ptr(rows), _lib.ptr(n),
                               T, HID, float(eps), _lib.ptr(parts) if np_ else None, parts.stride(0) if np_ else 0, np_,
                               _lib.ptr(pending.a_s) if np_ else None, _lib.ptr(pending.w_s) if np_ else None,
                               _lib.stream())
    _lib.check(rc, f"norm_q8 T={T} HID={HID} parts={np_}")


def gated_norm_q8(o, proj, z_off, w, inv_s, q, s, n, T, cfg, mode=0, amax=None, sync=None):
    """The gated RMSNorm of the linear-attention output + per-token int8 (the reference's gated_norm_q8,
    kernels/quant.py:460-470): o fp32 [>= T, v_heads * gdn_dim], the gate z = proj[:, z_off : z_off + v_heads * gdn_dim]
    (bf16, proj's row stride honoured), w fp32 [gdn_dim], inv_s fp32 [v_heads * gdn_dim] -> q int8, s fp32 [>= T].
    cfg: anything with v_heads, gdn_dim, eps.  Modes as rows_q8."""
    HV, D = cfg.v_heads, cfg.gdn_dim
    _lib.need_cuda(o, proj, q, s, n)
    amax = _mode_args(mode, amax, sync, T)
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape[1] != HV * D or proj.dtype != torch.bfloat16 \
            or proj.stride(1) != 1 or q.shape[1] != HV * D:
        raise RuntimeError("gated_norm_q8: o fp32 [T, v_heads * gdn_dim] contiguous, proj bf16 with unit column stride")
    if mode == 3:
        rc = _lib.lib().pb_gated_norm_q8_exchange(_lib.ptr(o), _lib.ptr(proj), proj.stride(0), int(z_off), _lib.ptr(w),
                                                  _lib.ptr(inv_s), _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), T, HV, D,
                                                  float(cfg.eps), ctypes.byref(_sync_struct(sync)), _lib.stream())
    else:
        rc = _lib.lib().pb_gated_norm_q8(_lib.ptr(o), _lib.ptr(proj), proj.stride(0), int(z_off), _lib.ptr(w),
                                         _lib.ptr(inv_s), _lib.ptr(q), _lib.ptr(s), _lib.ptr(n), T, HV, D, float(cfg.eps),
                                         mode, _lib.ptr(amax), _lib.stream())
    _lib.check(rc, f"gated_norm_q8 T={T} heads={HV} dim={D} mode={mode}")


def rows_g(x, q, s, xs, n, T):
    """x bf16 / fp32 [>= T, K] -> q int8 [M, K], s fp32 [K/256, M], xs int8 [K/256, M, 16] (super-block-major)."""
    K = q.shape[1]
    Ma = s.shape[1]
    _lib.need_cuda(x, q, s, xs, n)
    if x.dtype not in (torch.bfloat16, torch.float32) or not x.is_contiguous() or x.shape[1] != K:
        raise RuntimeError("rows_g: x must be contiguous bf16 / fp32 [T, K]")
    if s.shape[0] != K // 256 or xs.shape != (K // 256, Ma, 16) or not s.is_contiguous() or not xs.is_contiguous():
        raise RuntimeError("rows_g: s must be [K/256, M] and xs [K/256, M, 16], contiguous")
    rc = _lib.lib().pb_quant_g(_lib.ptr(x), int(x.dtype == torch.float32), _lib.ptr(q), _lib.ptr(s), _lib.ptr(xs),
                               _lib.ptr(n), T, Ma, K, _lib.stream())
    _lib.check(rc, f"rows_g T={T} K={K}")


def _g_outputs(q, s, xs, K, what):
    Ma = s.shape[1]
    if K % 256 or q.shape[1] != K or s.shape[0] != K // 256 or xs.shape != (K // 256, Ma, 16) or not q.is_contiguous() \
            or not s.is_contiguous() or not xs.is_contiguous():
        raise RuntimeError(f"{what}: q int8 [M, K], s fp32 [K/256, M], xs int8 [K/256, M, 16], contiguous, K % 256 == 0")
    return Ma


def swiglu_g(gu, q, s, xs, n, T):
    """SwiGLU into the W4A8 activation triple (the reference's swiglu_g, kernels/quant.py:407-409): gu bf16
    [>= T, 2 FF] -> q int8 [M, FF], s fp32 [FF/256, M], xs int8 [FF/256, M, 16]."""
    FF = q.shape[1]
    _lib.need_cuda(gu, q, s, xs, n)
    Ma = _g_outputs(q, s, xs, FF, "swiglu_g")
    if gu.dtype != torch.bfloat16 or gu.shape[1] != 2 * FF or not gu.is_contiguous():
        raise RuntimeError("swiglu_g: gu must be contiguous bf16 [T, 2 FF]")
    rc = _lib.lib().pb_swiglu_g(_lib.ptr(gu), _lib.ptr(q), _lib.ptr(s), _lib.ptr(xs), _lib.ptr(n), T, Ma, FF, _lib.stream())
    _lib.check(rc, f"swiglu_g T={T} FF={FF}")


def norm_g(h, w, q, s, xs, n, T, eps):
    """RMSNorm into the W4A8 activation triple (the reference's norm_g, kernels/quant.py:397-399)."""
    HID = h.shape[1]
    _lib.need_cuda(h, w, q, s, xs, n)
    Ma = _g_outputs(q, s, xs, HID, "norm_g")
    if h.dtype != torch.float32 or not h.is_contiguous():
        raise RuntimeError("norm_g: h must be contiguous fp32 [T, HID]")
    rc = _lib.lib().pb_norm_g(_lib.ptr(h), _lib.ptr(w), _lib.ptr(q), _lib.ptr(s), _lib.ptr(xs), _lib.ptr(n), T, Ma, HID,
                              float(eps), _lib.stream())
    _lib.check(rc, f"norm_g T={T} HID={HID}")


def gated_norm_g(o, proj, z_off, w, q, s, xs, n, T, cfg):
    """The gated norm into the W4A8 activation triple (the reference's gated_norm_g, kernels/quant.py:402-404)."""
    HV, D = cfg.v_heads, cfg.gdn_dim
    _lib.need_cuda(o, proj, q, s, xs, n)
    Ma = _g_outputs(q, s, xs, HV * D, "gated_norm_g")
    if o.dtype != torch.float32 or not o.is_contiguous() or proj.dtype != torch.bfloat16 or proj.stride(1) != 1:
        raise RuntimeError("gated_norm_g: o fp32 contiguous, proj bf16 with unit column stride")
    rc = _lib.lib().pb_gated_norm_g(_lib.ptr(o), _lib.ptr(proj), proj.stride(0), int(z_off), _lib.ptr(w), _lib.ptr(q),
                                    _lib.ptr(s), _lib.ptr(xs), _lib.ptr(n), T, Ma, HV, D, float(cfg.eps), _lib.stream())
    _lib.check(rc, f"gated_norm_g T={T} heads={HV} dim={D}")


def fold(h, parts, pending, n, T):
    """Finish a deferred residual add (w8a8.Deferred) in h fp32 [>= T, N]: h += (float(sum of slots) * a_s) * w_s with
    the unsplit epilogue's roundings.  parts: the int32 slots [S, rows, N] unless the Deferred names its own."""
    if not pending:
        return
    if pending.parts is not None:
        parts = pending.parts
    _lib.need_cuda(h, parts, n)
    N = h.shape[1]
    if h.dtype != torch.float32 or parts.dtype != torch.int32 or parts.shape[2] != N or h.stride(1) != 1:
        raise RuntimeError("fold: h fp32 [T, N], parts int32 [S, rows, N]")
    if pending.sync is not None:
        # every rank's slots, read by the kernel itself after a flag handshake (kernels/quant.py:128-141, :434-457)
        rc = _lib.lib().pb_fold_sync(_lib.ptr(h), h.stride(0), _lib.ptr(parts), parts.stride(0), pending.n,
                                     _lib.ptr(pending.a_s), _lib.ptr(pending.w_s), _lib.ptr(n), T, N,
                                     ctypes.byref(_sync_struct(pending.sync)), _lib.stream())
        _lib.check(rc, f"fold T={T} N={N} S={pending.n} over {pending.sync.world} ranks")
        return
    rc = _lib.lib().pb_fold(_lib.ptr(h), h.stride(0), _lib.ptr(parts), parts.stride(0), pending.n,
                            _lib.ptr(pending.a_s), _lib.ptr(pending.w_s), _lib.ptr(n), T, N, _lib.stream())
    _lib.check(rc, f"fold T={T} N={N} S={pending.n}")
