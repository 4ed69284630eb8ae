"""W4A8 projections on a Q4_K_M file's own weights: the operator API of the reference's kernels/w4a8.py over the
sm_100a library.

    W4                         a repacked k-quant matrix                                   (w4a8.py:44-67)
    repack(kq)                 KQuant (Q4_K / Q6_K raw super-blocks) -> W4                 (w4a8.py:70-94)
    concat, segments, seg_rows, seg_width, gemm_segs   fused projections of mixed kinds    (w4a8.py:97-140)
    gemm(xq, a, xs, w, out, n_rows, epi)               the GEMM                            (w4a8.py:353-366)

Layouts (the GEMM kernel reads exactly these):
  Q4_K  q uint8 [n, k/2]: per 32 inputs 16 bytes, byte t = q[t] | q[t + 16] << 4; sc, mn uint8 [k/256, n, 8] (the 6-bit
        sub-block scales and mins, super-block-major); d, dm fp32 [k/256, n].
  Q6_K  q int8 [n, k] (value - 32); sc int8 [k/256, n, 16]; d fp32 [k/256, n].
Activations come from quant.rows_g: xq int8 [M, k], a fp32 [k/256, M], xs int8 [k/256, M, 16].
The arithmetic is the reference's (w4a8.py:14-24): integer inside a 256-input super-block, one fp32 step per
super-block, the same bits for every kernel shape and batch.
"""
from __future__ import annotations

from typing import NamedTuple

import torch

from . import _lib
from . import gguf_weights as GW

QK_K = 256


class W4(NamedTuple):
    kind: str               # "q4k" or "q6k"
    q: torch.Tensor
    sc: torch.Tensor
    mn: torch.Tensor        # q6k: None
    d: torch.Tensor
    dm: torch.Tensor        # q6k: None
    n: int
    k: int

    @property
    def shape(self):
        return (self.n, self.k)

    def rows(self, r0, r1):
        """Rows r0:r1: the values a view, the super-block-major scales copied (the GEMM reads them contiguous)."""
        cut = lambda t: None if t is None else t[:, r0:r1].contiguous()     # noqa: E731
        return W4(self.kind, self.q[r0:r1], cut(self.sc), cut(self.mn), cut(self.d), cut(self.dm), r1 - r0, self.k)

    def to(self, device):
        mv = lambda t: None if t is None else t.to(device)                   # noqa: E731
        return W4(self.kind, mv(self.q), mv(self.sc), mv(self.mn), mv(self.d), mv(self.dm), self.n, self.k)

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.q, self.sc, self.mn, self.d, self.dm) if t is not None)


def repack(kq: GW.KQuant) -> W4:
    """A KQuant matrix (any device) -> W4."""
    raw = kq.raw
    n, nb = raw.shape[0], raw.shape[1]
    blocks = raw.reshape(n * nb, raw.shape[2])
    major = lambda t: t.reshape(n, nb, -1).transpose(0, 1).contiguous()     # noqa: E731  [n, nb, x] -> [nb, n, x]
    if kq.type == GW.GGML_Q4_K:
        d = blocks[:, 0:2].contiguous().view(torch.float16).float().reshape(n, nb)
        dm = blocks[:, 2:4].contiguous().view(torch.float16).float().reshape(n, nb)
        sc, mn = GW.scale_min_k4(blocks[:, 4:16])
        # ggml keeps two sub-blocks per 32 bytes (low nibbles, high nibbles); regroup per sub-block of 32 inputs and
        # pair input t with input t + 16 in one byte
        v = blocks[:, 16:144].to(torch.int32).reshape(-1, 4, 32)
        v = torch.stack([v & 15, v >> 4], 2).reshape(n, nb * 8, 32)
        q = (v[..., :16] | (v[..., 16:] << 4)).to(torch.uint8).reshape(n, kq.k // 2)
        return W4("q4k", q.contiguous(), major(sc.to(torch.uint8)), major(mn.to(torch.uint8)), d.t().contiguous(),
                  dm.t().contiguous(), n, kq.k)
    if kq.type == GW.GGML_Q6_K:
        q = (GW.q6k_values(blocks) - 32).to(torch.int8).reshape(n, kq.k)
        sc = blocks[:, 192:208].contiguous().view(torch.int8)
        d = blocks[:, 208:210].contiguous().view(torch.float16).float().reshape(n, nb)
        return W4("q6k", q.contiguous(), major(sc), None, d.t().contiguous(), None, n, kq.k)
    raise ValueError(f"k-quant type {kq.type}: Q4_K and Q6_K are supported")


def concat(ws):
    """Stack W4 matrices of ONE kind on top of each other (the rows of a fused projection).  The quants are row-major
    and grow along dim 0; scales, mins and d are stored super-block-major [k/256, n, ...] and grow along dim 1."""
    first = ws[0]
    odd = sorted({w.kind for w in ws} - {first.kind})
    if odd:
        raise ValueError(f"one fused segment holds one k-quant kind: {first.kind} cannot take {odd}")

    def joined(field, dim):
        parts = [getattr(w, field) for w in ws]
        return None if parts[0] is None else torch.cat(parts, dim)
    return W4(first.kind, joined("q", 0), joined("sc", 1), joined("mn", 1), joined("d", 1), joined("dm", 1),
              sum(w.n for w in ws), first.k)


def segments(kqs, device):
    """The matrices of a fused projection, top to bottom (e.g. q, k, v of a Q4_K_M file: Q4_K, Q4_K, Q6_K), as
    [(W4, its first output column)].  Runs of neighbours that share a kind become one W4, so the projection costs one
    GEMM per kind change, not one per matrix."""
    runs = []
    for kq in kqs:
        if not isinstance(kq, GW.KQuant):
            raise ValueError(f"W4A8 runs on k-quant matrices; a {type(kq).__name__} was given")
        w = repack(kq.to(device))
        if runs and runs[-1][0].kind == w.kind:
            runs[-1].append(w)
        else:
            runs.append([w])
    out, column = [], 0
    for run in runs:
        w = run[0] if len(run) == 1 else concat(run)
        out.append((w, column))
        column += w.n
    return out


def seg_rows(segs, r0, r1):
    """The part of a fused projection that produces output columns [r0, r1): each segment cut to its overlap with
    the range, first columns renumbered from r0 (a tensor-parallel rank's slice, or a head's rows)."""
    picked = []
    for w, first in segs:
        lo, hi = max(r0 - first, 0), min(r1 - first, w.n)
        if hi > lo:
            picked.append((w.rows(lo, hi), first + lo - r0))
    return picked


def seg_width(segs):
    """Output columns of a fused projection."""
    return max(first + w.n for w, first in segs)


def gemm_segs(xq, a, xs, segs, out, n_rows, epi=0, pdl=0):
    """The fused projection's GEMMs: every segment writes (or adds into) its own column range of `out`."""
    for w, first in segs:
        gemm(xq, a, xs, w, out[:, first:first + w.n], n_rows, epi, pdl=pdl)


def pick_split(M, N, K, tile=128):
    """K splits of the few-rows kernels (M <= 16): one CTA per SM, so the time goes as (waves of CTAs) / (slices):
    the slice count that makes that smallest, at least four super-blocks per slice, the fewest slices among equals.
    Exact (the per-super-block terms meet in a workspace): always on."""
    if M > 16:
        return 1
    tiles = -(-N // tile)
    best, cost = 1, float(-(-tiles // 148))
    for s in range(2, min(8, (K // 256) // 4) + 1):
        c = -(-tiles * s // 148) / s
        if c < cost - 1e-9:
            best, cost = s, c
    return best


def gemm(xq, a, xs, w: W4, out, n_rows, epi=0, cfg=None, pdl=0):
    """xq int8 [M, K], a fp32 [K/256, M], xs int8 [K/256, M, 16], w W4 [N, K] -> out [M, N]: bf16 (epi 0) or added
    into fp32 (epi 1); out may be a column slice.  cfg: None (pick) or the number of K splits of the few-rows Q4_K kernel
    (Q4_K and Q6_K, M <= 16; exact: the same bits for every split); pdl is accepted for signature parity."""
    M, K = xq.shape
    _lib.need_cuda(xq, a, w.q, out, n_rows)
    if K != w.k or a.shape[0] != K // QK_K or not xq.is_contiguous() or not a.is_contiguous():
        raise RuntimeError("w4a8.gemm: xq [M, K] int8 contiguous, a [K/256, M] fp32 contiguous")
    want = torch.bfloat16 if epi == 0 else torch.float32
    if out.dtype != want or out.shape[1] != w.n or out.stride(1) != 1 or out.shape[0] < M:
        raise RuntimeError(f"w4a8.gemm: out must be {want} [>= {M}, {w.n}] with unit column stride")
    q4 = w.kind == "q4k"
    if q4 and (xs is None or xs.shape[1] != a.shape[1] or not xs.is_contiguous()):
        raise RuntimeError("w4a8.gemm: Q4_K needs the activation group sums xs [K/256, M, 16]")
    for t in (w.q, w.sc, w.mn, w.d, w.dm):
        if t is not None and not t.is_contiguous():
            raise RuntimeError("w4a8.gemm: W4 tensors must be contiguous (W4.rows copies the scales)")
    split = pick_split(M, w.n, K, 128 if q4 else 64) if cfg is None else max(1, int(cfg))
    ws = counters = None
    if split > 1 and M <= 16:
        from . import w8a8 as KW
        ws, counters = KW._workspace(xq.device)
        if _lib.lib().pb_w4a8_workspace_bytes(M, w.n, K) > ws.numel():
            split, ws, counters = 1, None, None
    else:
        split = 1
    rc = _lib.lib().pb_w4a8_gemm(_lib.ptr(xq), _lib.ptr(a), _lib.ptr(xs) if q4 else None, a.shape[1], 0 if q4 else 1,
                                 _lib.ptr(w.q), _lib.ptr(w.sc), _lib.ptr(w.mn), _lib.ptr(w.d), _lib.ptr(w.dm),
                                 _lib.ptr(out), out.stride(0), _lib.ptr(n_rows), M, w.n, K, epi, split, _lib.ptr(ws),
                                 0 if ws is None else ws.numel(), _lib.ptr(counters),
                                 0 if counters is None else counters.numel(), _lib.stream())
    _lib.check(rc, f"w4a8 gemm {w.kind} M={M} N={w.n} K={K} epi={epi}")
