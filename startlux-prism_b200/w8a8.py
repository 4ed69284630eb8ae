"""W8A8 projections: the operator API of the reference's kernels/w8a8.py over the sm_100a library.

    gemm(a, a_s, w, w_s, out, n_rows, gk, epi=0, ...)   int8 x int8 GEMM with scale epilogues     (w8a8.py:183-231)
    gemm_i32(a, a_s, w, w_s, slots, n_rows, ...)        raw int32 sums of a tensor-parallel shard (w8a8.py:234-261)
    quant_rows(x, gk, n_rows)                           symmetric int8 per (row, group)           (w8a8.py:264-271)
    weight_from_q8(q8, gk, smooth)                      Q8_0 -> (int8, fp32 scales)               (w8a8.py:274-286)
    interleave_gate_up(gate, up, bn)                                                              (w8a8.py:289-294)
    Deferred                                            a residual add left to quant.fold         (w8a8.py:171-180)

gk == K (the engine's mode): one scale per token and per output channel; every kernel, K split and batch size gives an
output element the same bits: v = (float(acc) * a_s[m]) * w_s[n], each product rounded, epi 1 adds with one more
rounding.  gk == 32 uses Q8_0's own block scales: fp32 partial products added in group order.
Kernel choice (this module's table replaces the reference's per-GPU JSON tables): more than 64 rows -> the persistent
128 x 256 tile kernel; up to 64 rows -> the operand-swapped split-K kernel, the splits' int32 sums either deferred to
the caller's `slots` (epi 1) or added inside the kernel through a workspace.
"""
from typing import NamedTuple

import torch

from . import _lib

EPI_BF16, EPI_ADD, EPI_SWIGLU, EPI_I32, EPI_F32 = 0, 1, 2, 3, 4
FEW_ROWS = 64                    # up to this many rows the operand-swapped kernel runs
MAX_SPLIT = 8
RESIDENT_CTAS = 296              # two CTAs of the few-rows kernel per SM on 148 SMs
SM_COUNT = 148
WS_BYTES = 96 << 20              # split-K workspace per device (allocated at the first call that needs it)

_WORKSPACE = {}


class Deferred(NamedTuple):
    """A residual add left to the next reader of the residual (quant.fold / quant.norm_q8): `n` int32 slots of partial
    sums and the projection's scales; `parts` names the slots when they are not the reader's own buffer; `sync` (a
    quant.Sync from tp.Group.sync()): the slots are this rank's only and the reader adds every rank's itself, over
    NVLink, after a flag handshake."""
    n: int
    a_s: torch.Tensor
    w_s: torch.Tensor
    parts: torch.Tensor = None
    sync: object = None


def _workspace(device):
    """(workspace bytes tensor, zeroed int32 counters) of a device; allocated once, outside any graph capture.  One
    array per device, shared by the W8A8, W4A8 and MXFP4 split-K kernels on whatever stream calls them: two products
    that split K and overlap on the GPU (different streams) race on it - keep split-K products of one device on one
    stream, or give the second stream its own arrays through the C entry points."""
    key = torch.device(device).index or 0
    if key not in _WORKSPACE:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the split-K workspace must exist before graph capture: run the GEMM once eagerly")
        _WORKSPACE[key] = (torch.empty(WS_BYTES, dtype=torch.uint8, device=device),
                           torch.zeros(65536, dtype=torch.int32, device=device))
    return _WORKSPACE[key]


def _workspace_if_ready(device):
    """The device's workspace when it exists or may be allocated now (not during graph capture), else (None, None):
    for uses that are an optimisation, not a need (the many-rows kernel's split of its last, partial wave of tiles)."""
    key = torch.device(device).index or 0
    if key not in _WORKSPACE and torch.cuda.is_current_stream_capturing():
        return None, None
    return _workspace(device)


def reset_workspace(device=None):
    """Zero the split-K arrival counters (after a kernel reported PB_DEVICE_TIMEOUT: a CTA that gave up a wait did not
    count itself in, so its tile's counter is left non-zero)."""
    for key, (_, counters) in _WORKSPACE.items():
        if device is None or key == (torch.device(device).index or 0):
            counters.zero_()


GEMV_ROWS = 1        # gk == K: this many rows against few weight rows run on the CUDA cores (PB_W8A8_GEMV_ROWS)


def pick_split(M, N, K, limit=MAX_SPLIT):
    """K splits.  Few rows (operand-swapped kernel): as many CTAs as stay resident together, at least two 128-byte K
    blocks each.  Many rows (tile kernel, one CTA per SM): only when the 128 x 256 tiles leave most SMs idle and K is
    long (at least 32 K blocks per slice; measured: a gain for K = 17408 at 128-256 rows, a loss for K = 5120) - the
    slices' int32 sums meet in the workspace, exactly."""
    kb = -(-K // 128)
    if M > FEW_ROWS:
        tiles = -(-M // 128) * -(-N // 256)
        if N <= 128 or tiles * 2 <= SM_COUNT:                    # the library's rule: narrower tiles when they are few
            tiles = -(-M // 128) * -(-N // 128)
        return max(1, min(limit, SM_COUNT // tiles, kb // 32))
    tiles = -(-N // 128)
    return max(1, min(limit, RESIDENT_CTAS // tiles, kb // 2))


_TABLE = None


def _choice(M, N, K, residual):
    """The measured choice for this projection shape at the nearest measured row count (tune.py's table), or None."""
    global _TABLE
    if _TABLE is None:
        from . import tune
        _TABLE = tune.load_table()
    by_m = _TABLE.get((N, K, bool(residual)))
    if not by_m:
        return None
    import math
    # the one-row entry was measured on the CUDA-core kernel: it says nothing about the tensor-core kernel at 2+ rows
    rows = [x for x in by_m if x > GEMV_ROWS] if M > GEMV_ROWS else list(by_m)
    if not rows:
        return None
    m = min(rows, key=lambda x: abs(math.log(x) - math.log(max(M, 1))))
    return by_m[m]


def effective_split(K, split):
    """The K splits the few-rows kernel really runs for a request of `split`: whole 128-byte K blocks per slice, no
    empty slice (the library applies the same rule)."""
    kb = -(-K // 128)
    split = max(1, min(split, kb))
    per = -(-kb // split)
    return -(-kb // per)


def _call(a, a_s, w, w_s, out, ldo, n_rows, gk, epi, split, slot_stride=0, ws=None, counters=None, pdl=False):
    M, K = a.shape
    N = w.shape[0]
    _lib.need_cuda(a, w, out, n_rows)
    if a.dtype != torch.int8 or w.dtype != torch.int8 or not a.is_contiguous() or not w.is_contiguous():
        raise RuntimeError("w8a8.gemm: a and w must be contiguous int8 [rows, K]")
    if w.shape[1] != K:
        raise RuntimeError(f"w8a8.gemm: K mismatch ({K} vs {w.shape[1]})")
    if n_rows.dtype != torch.int32:
        raise RuntimeError("w8a8.gemm: n_rows must be a device int32 tensor")
    rc = _lib.lib().pb_w8a8_gemm(_lib.ptr(a), _lib.ptr(a_s), _lib.ptr(w), _lib.ptr(w_s), _lib.ptr(out), ldo,
                                 _lib.ptr(n_rows), M, N, K, gk, epi, split, slot_stride, _lib.ptr(ws),
                                 0 if ws is None else ws.numel(), _lib.ptr(counters),
                                 0 if counters is None else counters.numel(), int(bool(pdl)), _lib.stream())
    _lib.check(rc, f"w8a8 gemm M={M} N={N} K={K} gk={gk} epi={epi} split={split}")


def _scales_ok(s, rows, groups, what):
    if s.dtype != torch.float32 or s.numel() != rows * groups or not s.is_contiguous():
        raise RuntimeError(f"w8a8.gemm: {what} must be contiguous fp32 with {rows} x {groups} elements")


def gemm(a, a_s, w, w_s, out, n_rows, gk, epi=0, outs=None, cfg=None, slots=None, pdl=False):
    """a int8 [M, K], a_s fp32 [M, K/gk], w int8 [N, K], w_s fp32 [N, K/gk] -> out: bf16 [M, N] (epi 0) or added into
    fp32 [M, N] (epi 1); out may be a column slice of a wider buffer (its row stride is honoured).  Returns a Deferred
    when an epi 1 product split K into `slots` (int32 [S, rows, N]), else None.  cfg: None or the number of K splits.
    pdl: the few-rows kernel is launched as a programmatic dependent of the kernel before it on the stream: its
    weights stream while that kernel (the producer of a and a_s) still runs; everything else waits for it."""
    M, K = a.shape
    N = w.shape[0]
    if epi == EPI_SWIGLU:
        return _gemm_swiglu(a, a_s, w, w_s, out, n_rows, gk, outs, cfg)
    if epi not in (EPI_BF16, EPI_ADD, EPI_F32) or (epi == EPI_F32 and (gk != 32 or M > FEW_ROWS)):
        raise ValueError(f"epi {epi}")                 # EPI_F32 (plain fp32 store): the vocabulary head, decode.head_q8
    want = torch.bfloat16 if epi == EPI_BF16 else torch.float32
    if out.dtype != want or out.shape[0] < M or out.shape[1] != N or out.stride(1) != 1:
        raise RuntimeError(f"w8a8.gemm: out must be {want} [>= {M}, {N}] with unit column stride")
    _scales_ok(a_s, M, K // gk, "a_s")
    _scales_ok(w_s, N, K // gk, "w_s")
    if gk != K and gk != 32:
        # any other group size: one kernel shape, groups added in order, no K split
        _call(a, a_s, w, w_s, out, out.stride(0), n_rows, gk, epi, 1)
        return None
    if gk != K:
        # Q8_0's own scales: one K slice keeps the reference's group order (bit-exact); cfg = K splits (few rows only)
        # trades that for parallelism: slices added in slice order, within one bf16 step of the unsplit result
        split = effective_split(K, int(cfg)) if cfg is not None and M <= FEW_ROWS else 1
        ws = counters = None
        if split > 1:
            ws, counters = _workspace(a.device)
        _call(a, a_s, w, w_s, out, out.stride(0), n_rows, gk, epi, split, 0, ws, counters, pdl=pdl)
        return None
    if cfg is None and not pdl and K % 256 == 0 and M <= GEMV_ROWS and (N + 7) // 8 < 8 * SM_COUNT:
        # one row against few weight rows: the library's CUDA-core kernel (no K split: its CTAs already cover the SMs); same bits
        _call(a, a_s, w, w_s, out, out.stride(0), n_rows, gk, epi, 1)
        return None
    defer_ok = True
    if cfg is not None:
        split = int(cfg)
    else:
        c = _choice(M, N, K, epi == EPI_ADD) if M <= FEW_ROWS else None
        split = c["split"] if c else pick_split(M, N, K)
        defer_ok = c["defer"] if c else True
    split = effective_split(K, split)
    if split > 1 and M <= FEW_ROWS and epi == EPI_ADD and slots is not None and slots.shape[1] >= M and defer_ok:
        split = effective_split(K, min(split, slots.shape[0]))
        if split > 1:
            _check_slots(slots, M, N)
            _call(a, a_s, w, w_s, slots, N, n_rows, gk, EPI_I32, split, slots.stride(0), pdl=pdl)
            return Deferred(split, a_s, w_s)
    ws = counters = None
    if split > 1:
        ws, counters = _workspace(a.device)
        while split > 1 and _lib.lib().pb_w8a8_workspace_bytes(M, N, split) > ws.numel():
            split -= 1
        if split == 1:
            ws = counters = None
    if split == 1 and M > FEW_ROWS:
        ws, counters = _workspace_if_ready(a.device)     # lets the kernel split the K range of a partial last wave
    _call(a, a_s, w, w_s, out, out.stride(0), n_rows, gk, epi, split, 0, ws, counters, pdl=pdl)
    return None


def _gemm_swiglu(a, a_s, w, w_s, out, n_rows, gk, outs, cfg):
    """epi 2 (kernels/w8a8.py:86-98): w is interleave_gate_up(gate, up, bn) (w_s in the same row order); out int8
    [M, FF] = silu(gate) * up quantized per row and tile of bn / 2 columns, outs fp32 [M, 2 FF / bn] the scales: the
    input of a down projection with gk = bn / 2.  cfg: bn itself, or the reference's config tuple (bn = cfg[1]);
    default 128."""
    M, K = a.shape
    N = w.shape[0]
    bn = 128 if cfg is None else int(cfg[1] if isinstance(cfg, (tuple, list)) else cfg)
    if gk != K:
        raise RuntimeError("w8a8.gemm epi 2: one scale group over K (gk == K)")
    if outs is None or outs.dtype != torch.float32 or not outs.is_contiguous() or outs.numel() < M * (N // bn) \
            or outs.shape[-1] != N // bn:
        raise RuntimeError(f"w8a8.gemm epi 2: outs must be contiguous fp32 [>= {M}, {N // bn}]")
    if out.dtype != torch.int8 or out.shape[0] < M or out.shape[1] != N // 2 or out.stride(1) != 1:
        raise RuntimeError(f"w8a8.gemm epi 2: out must be int8 [>= {M}, {N // 2}]")
    _lib.need_cuda(a, w, out, outs, n_rows)
    if a.dtype != torch.int8 or w.dtype != torch.int8 or not a.is_contiguous() or not w.is_contiguous() or w.shape[1] != K:
        raise RuntimeError("w8a8.gemm: a and w must be contiguous int8 [rows, K]")
    _scales_ok(a_s, M, 1, "a_s")
    _scales_ok(w_s, N, 1, "w_s")
    rc = _lib.lib().pb_w8a8_gemm_swiglu(_lib.ptr(a), _lib.ptr(a_s), _lib.ptr(w), _lib.ptr(w_s), _lib.ptr(out),
                                        out.stride(0), _lib.ptr(outs), _lib.ptr(n_rows), M, N, K, bn, _lib.stream())
    _lib.check(rc, f"w8a8 gemm epi 2 M={M} N={N} K={K} bn={bn}")
    return None


def _check_slots(slots, M, N):
    if slots.dtype != torch.int32 or slots.dim() != 3 or slots.shape[1] < M or slots.shape[2] != N \
            or slots.stride(2) != 1 or slots.stride(1) != N:
        raise RuntimeError("slots must be int32 [S, rows >= M, N], rows contiguous")


def gemm_i32(a, a_s, w, w_s, slots, n_rows, max_split=4, pdl=False, split=None):
    """The int32 products a w^T without the scales into slots (int32 [S, rows, N]): a row-parallel shard's partial
    sums, added over the ranks (exact) and scaled later (Deferred, quant.fold).  Returns the number of slots written
    (K splits, at most max_split and slots.shape[0])."""
    M, K = a.shape
    N = w.shape[0]
    _check_slots(slots, M, N)
    S = split if split is not None else pick_split(M, N, K, min(max_split, slots.shape[0]))
    if M > FEW_ROWS:
        # many rows: one slot; K splits (when the tiles are few) meet in the workspace, exactly
        inner = effective_split(K, pick_split(M, N, K) if split is None else split)
        ws = counters = None
        if inner > 1:
            ws, counters = _workspace(a.device)
            if _lib.lib().pb_w8a8_workspace_bytes(M, N, inner) > ws.numel():
                inner, ws, counters = 1, None, None
        if inner == 1:
            ws, counters = _workspace_if_ready(a.device)
        _call(a, a_s, w, w_s, slots, N, n_rows, K, EPI_I32, inner, slots.stride(0), ws, counters, pdl=pdl)
        return 1
    S = effective_split(K, max(1, min(S, max_split, slots.shape[0])))
    _call(a, a_s, w, w_s, slots, N, n_rows, K, EPI_I32, S, slots.stride(0), pdl=pdl)
    return S


def gemm_scatter(a, w, blocks, block_rows, ldo, n_rows):
    """The int32 products a w^T of a row-parallel shard, written where they will be folded: output rows
    [o * block_rows, (o + 1) * block_rows) go to the device address blocks[o] (int32 [block_rows, N], row stride ldo),
    which may be another GPU's memory (tp.PeerBuffer): the tile kernel stores them over NVLink as it drains each tile.
    More than 64 rows, block_rows a multiple of 128, at most 8 blocks."""
    import ctypes
    M, K = a.shape
    N = w.shape[0]
    _lib.need_cuda(a, w, n_rows)
    if a.dtype != torch.int8 or w.dtype != torch.int8 or w.shape[1] != K or not a.is_contiguous() or not w.is_contiguous():
        raise RuntimeError("gemm_scatter: a int8 [M, K], w int8 [N, K], contiguous")
    arr = (ctypes.c_void_p * len(blocks))(*[int(b) for b in blocks])
    rc = _lib.lib().pb_w8a8_gemm_scatter(_lib.ptr(a), _lib.ptr(w), arr, len(blocks), block_rows, ldo, _lib.ptr(n_rows),
                                         M, N, K, _lib.stream())
    _lib.check(rc, f"w8a8 gemm_scatter M={M} N={N} K={K} blocks={len(blocks)}x{block_rows}")


def quant_rows(x, gk, n_rows=None):
    """x [M, K] bf16 / fp32 -> (int8 [M, K], fp32 scales [M, K / gk]), symmetric per group of gk inputs."""
    M, K = x.shape
    _lib.need_cuda(x)
    q = torch.empty(M, K, dtype=torch.int8, device=x.device)
    s = torch.empty(M, K // gk, dtype=torch.float32, device=x.device)
    if n_rows is None:
        n_rows = torch.tensor([M], dtype=torch.int32, device=x.device)
    if x.dtype not in (torch.bfloat16, torch.float32) or not x.is_contiguous():
        raise RuntimeError("quant_rows: x must be contiguous bf16 or fp32")
    rc = _lib.lib().pb_quant_rows(_lib.ptr(x), int(x.dtype == torch.float32), K, None, _lib.ptr(q), _lib.ptr(s),
                                  _lib.ptr(n_rows), M, K, gk, 0, None, _lib.stream())
    _lib.check(rc, f"quant_rows M={M} K={K} gk={gk}")
    return q, s


def weight_from_q8(q8, gk, smooth=None):
    """Q8_0 matrix -> (int8 [N, K], fp32 scales [N, K / gk]).  gk == 32 without smoothing keeps the file's values and
    block scales; otherwise the dequantized weights (times smooth[k], SmoothQuant) are quantized again per group:
    s = max|g| / 127 (at least 1e-10 / 127), q = round(g / s) clamped to +-127.  Load-time, plain torch, any device."""
    if gk == 32 and smooth is None:
        return q8.qs.contiguous(), q8.d.float().contiguous()
    wf = q8.dequant(torch.float32)
    if smooth is not None:
        wf = wf * smooth[None, :]
    N, K = wf.shape
    g = wf.view(N, K // gk, gk)
    s = g.abs().amax(-1).clamp_min(1e-10) / 127.0
    q = torch.round(g / s[..., None]).clamp(-127, 127).to(torch.int8).view(N, K)
    return q.contiguous(), s.contiguous()


def interleave_gate_up(gate, up, bn):
    """Rows of gate [FF, K] and up [FF, K] -> [2 FF, K] in tiles of bn rows: bn / 2 gate rows then the same up rows."""
    FF, K = gate.shape
    h = bn // 2
    if FF % h:
        raise ValueError(f"FF {FF} is not a multiple of {h}")
    return torch.stack([gate.view(FF // h, h, K), up.view(FF // h, h, K)], 1).reshape(2 * FF, K).contiguous()


def l2_prefetch(tensors, ctas=32):
    """Request the bytes of up to eight contiguous tensors into L2 on the current stream (the reference's
    cuda_ext.l2_prefetch, kernels/cuda_ext.py:171-173; four tensors there).  Meant for a side stream while a
    latency-bound kernel runs; off by default everywhere in this package."""
    import ctypes
    tensors = list(tensors)
    if not 1 <= len(tensors) <= 8 or any(not t.is_cuda or not t.is_contiguous() for t in tensors):
        raise RuntimeError("l2_prefetch: one to eight contiguous CUDA tensors")
    ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    sizes = (ctypes.c_long * len(tensors))(*[t.numel() * t.element_size() for t in tensors])
    _lib.check(_lib.lib().pb_l2_prefetch(ptrs, sizes, len(tensors), int(ctas), _lib.stream()), "l2_prefetch")
