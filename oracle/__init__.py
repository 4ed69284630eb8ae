"""CPU oracle of the quantized linear-layer path: ctypes bindings of oracle.c.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by bench.py's CPU-baseline legs, never by the
product package.  Each wrapper takes and returns numpy arrays (bf16 travels as uint16 bit patterns).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    """Compile oracle.c into liboracle.so beside it (gcc, a second or two)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
    return _LIB


def _p(x):
    return None if x is None else ctypes.c_void_p(x.ctypes.data)


def _c(x, dt):
    x = np.ascontiguousarray(x)
    assert x.dtype == dt, (x.dtype, dt)
    return x


def bf16_bits(x32):
    """fp32 array -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x32, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(bits):
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def w8a8_gemm(a, a_s, w, w_s, gk, epi, live=None, out=None):
    """a int8 [M, K], a_s fp32 [M, K/gk], w int8 [N, K], w_s fp32 [N, K/gk].  epi 0 -> bf16 bits uint16 [M, N];
    epi 1 -> fp32 `out` += (a copy is returned); epi 3 -> int32 [M, N]; epi 4 -> fp32 [M, N] = the groups' sums with the
    last multiply and the add fused (the vocabulary head).  Rows >= live keep `out`'s values (zeros)."""
    M, K = a.shape
    N = w.shape[0]
    live = M if live is None else live
    dt = {0: np.uint16, 1: np.float32, 3: np.int32, 4: np.float32}[epi]      # 4: the vocabulary head's plain fp32 store
    o = np.zeros((M, N), dt) if out is None else np.array(out, dtype=dt, copy=True, order="C")
    lib().orc_w8a8_gemm(_p(_c(a, np.int8)), _p(_c(a_s, np.float32)), _p(_c(w, np.int8)), _p(_c(w_s, np.float32)),
                        _p(o), ctypes.c_long(N), live, N, K, gk, epi)
    return o


def w8a8_swiglu_epi(a, a_s, w, w_s, bn, live=None):
    """The GEMM's fused SwiGLU epilogue on interleaved gate|up rows (tiles of bn): a int8 [M, K], a_s fp32 [M], w int8
    [N, K], w_s fp32 [N] -> (q int8 [M, N / 2], s fp32 [M, N / bn])."""
    M, K = a.shape
    N = w.shape[0]
    live = M if live is None else live
    q = np.zeros((M, N // 2), np.int8)
    s = np.zeros((M, N // bn), np.float32)
    lib().orc_w8a8_swiglu_epi(_p(_c(a, np.int8)), _p(_c(np.ravel(a_s), np.float32)), _p(_c(w, np.int8)),
                              _p(_c(np.ravel(w_s), np.float32)), _p(q), _p(s), live, N, K, bn)
    return q, s


def fold(h, slots, a_s, w_s, live=None):
    """h fp32 [rows, N] (a copy is returned), slots int32 [S, rows, N]."""
    h = np.array(h, dtype=np.float32, copy=True, order="C")
    slots = _c(slots, np.int32)
    S, rows, N = slots.shape
    live = h.shape[0] if live is None else live
    lib().orc_fold(_p(h), ctypes.c_long(N), _p(slots), ctypes.c_long(rows * N), S, _p(_c(a_s, np.float32)),
                   _p(_c(w_s, np.float32)), live, N)
    return h


def quant_rows(x, gk=None, inv_s=None, live=None, amax_in=None, want_amax=False):
    """x: bf16 bits (uint16) or fp32 [M, K] -> (q int8 [M, K], s fp32 [M, K/gk])."""
    M, K = x.shape
    gk = K if gk is None else gk
    live = M if live is None else live
    is_bf = x.dtype == np.uint16
    x = _c(x, np.uint16 if is_bf else np.float32)
    q = np.zeros((M, K), np.int8)
    s = np.zeros((M, K // gk), np.float32)
    am = np.zeros((M, K // gk), np.float32) if want_amax else None
    lib().orc_quant_rows(_p(x), int(is_bf), _p(None if inv_s is None else _c(inv_s, np.float32)), _p(q), _p(s), live,
                         K, gk, _p(None if amax_in is None else _c(amax_in, np.float32)), _p(am))
    return (q, s, am) if want_amax else (q, s)


def swiglu_q8(gu_bits, inv_s=None, live=None):
    M, F2 = gu_bits.shape
    FF = F2 // 2
    live = M if live is None else live
    q = np.zeros((M, FF), np.int8)
    s = np.zeros(M, np.float32)
    lib().orc_swiglu_q8(_p(_c(gu_bits, np.uint16)), _p(None if inv_s is None else _c(inv_s, np.float32)), _p(q), _p(s),
                        live, FF)
    return q, s


def norm_q8(h, w, eps, rows=None, live=None, parts=None, psa=None, psw=None):
    """h fp32 [R, HID] (updated in place when parts are given) -> (q int8 [T, HID], s fp32 [T])."""
    HID = h.shape[1]
    T = len(rows) if rows is not None else h.shape[0]
    live = T if live is None else live
    q = np.zeros((T, HID), np.int8)
    s = np.zeros(T, np.float32)
    assert h.dtype == np.float32 and h.flags["C_CONTIGUOUS"]
    n_parts = 0 if parts is None else parts.shape[0]
    lib().orc_norm_q8(_p(h), _p(_c(w, np.float32)), _p(q), _p(s), _p(None if rows is None else _c(rows, np.int32)), live,
                      HID, ctypes.c_float(eps), _p(None if parts is None else _c(parts, np.int32)),
                      ctypes.c_long(0 if parts is None else parts.shape[1] * parts.shape[2]), n_parts,
                      _p(None if psa is None else _c(psa, np.float32)), _p(None if psw is None else _c(psw, np.float32)))
    return q, s


def gated_norm_q8(o, proj_bits, z_off, w, inv_s, HV, D, eps, live=None, amax_in=None, want_amax=False):
    """o fp32 [T, HV * D], proj bf16 bits [T, P] -> (q int8 [T, HV * D], s fp32 [T][, amax fp32 [T]])."""
    T, P = proj_bits.shape
    live = T if live is None else live
    q = np.zeros((T, HV * D), np.int8)
    s = np.zeros(T, np.float32)
    am = np.zeros(T, np.float32)
    lib().orc_gated_norm_q8(_p(_c(o, np.float32)), _p(_c(proj_bits, np.uint16)), ctypes.c_long(P), ctypes.c_long(z_off),
                            _p(_c(w, np.float32)), _p(_c(inv_s, np.float32)), _p(q), _p(s), live, HV, D,
                            ctypes.c_float(eps), _p(None if amax_in is None else _c(amax_in, np.float32)), _p(am))
    return (q, s, am) if want_amax else (q, s)


def swiglu_g(gu_bits, live=None):
    """gu bf16 bits [T, 2 FF] -> the W4A8 activation triple of silu(gate) * up (quant_g of the fp32 row)."""
    T, F2 = gu_bits.shape
    live = T if live is None else live
    y = np.zeros((T, F2 // 2), np.float32)
    lib().orc_swiglu_y(_p(_c(gu_bits, np.uint16)), _p(y), live, F2 // 2)
    return quant_g(y, live)


def norm_g(h, w, eps, live=None):
    T, HID = h.shape
    live = T if live is None else live
    y = np.zeros((T, HID), np.float32)
    lib().orc_norm_y(_p(_c(h, np.float32)), _p(_c(w, np.float32)), _p(y), live, HID, ctypes.c_float(eps))
    return quant_g(y, live)


def gated_norm_g(o, proj_bits, z_off, w, HV, D, eps, live=None):
    T, P = proj_bits.shape
    live = T if live is None else live
    y = np.zeros((T, HV * D), np.float32)
    lib().orc_gated_norm_y(_p(_c(o, np.float32)), _p(_c(proj_bits, np.uint16)), ctypes.c_long(P), ctypes.c_long(z_off),
                           _p(_c(w, np.float32)), _p(y), live, HV, D, ctypes.c_float(eps))
    return quant_g(y, live)


def head_quant(h, w, eps, live=None):
    """h fp32 [B, HID] -> (q int8 [B, HID], s fp32 [B, HID / 32]): final RMSNorm + int8 per 32 inputs."""
    B, HID = h.shape
    live = B if live is None else live
    q = np.zeros((B, HID), np.int8)
    s = np.zeros((B, HID // 32), np.float32)
    lib().orc_head_quant(_p(_c(h, np.float32)), _p(_c(w, np.float32)), _p(q), _p(s), live, HID, ctypes.c_float(eps))
    return q, s


def quant_g(x, live=None):
    """x bf16 bits or fp32 [M, K] -> (q int8 [M, K], a fp32 [K/256, M], xs int8 [K/256, M, 16])."""
    M, K = x.shape
    live = M if live is None else live
    is_bf = x.dtype == np.uint16
    x = _c(x, np.uint16 if is_bf else np.float32)
    q = np.zeros((M, K), np.int8)
    a = np.zeros((K // 256, M), np.float32)
    xs = np.zeros((K // 256, M, 16), np.int8)
    lib().orc_quant_g(_p(x), int(is_bf), _p(q), _p(a), _p(xs), live, M, K)
    return q, a, xs


def w4a8_gemm(xq, a, xs, kind, wq, wsc, wmn, wd, wdm, epi=0, live=None, out=None):
    """Operands in the reference's W4 layout (kernels/w4a8.py:44-55); kind "q4k" or "q6k"."""
    M, K = xq.shape
    N = wq.shape[0]
    live = M if live is None else live
    dt = np.uint16 if epi == 0 else np.float32
    o = np.zeros((M, N), dt) if out is None else np.array(out, dtype=dt, copy=True, order="C")
    k4 = kind == "q4k"
    lib().orc_w4a8_gemm(_p(_c(xq, np.int8)), _p(_c(a, np.float32)), _p(_c(xs, np.int8)), a.shape[1],
                        _p(_c(wq, np.uint8 if k4 else np.int8)), _p(_c(wsc, np.uint8 if k4 else np.int8)),
                        _p(_c(wmn, np.uint8)) if k4 else None, _p(_c(wd, np.float32)),
                        _p(_c(wdm, np.float32)) if k4 else None, _p(o), ctypes.c_long(N), live, N, K,
                        0 if k4 else 1, epi)
    return o


def mxfp4_quant(x, inv=None, neg_zero=True):
    n, K = x.shape
    is_bf = x.dtype == np.uint16
    x = _c(x, np.uint16 if is_bf else np.float32)
    q = np.zeros((n, K // 2), np.uint8)
    s = np.zeros((n, K // 32), np.uint8)
    lib().orc_mxfp4_quant(_p(x), int(is_bf), _p(None if inv is None else _c(inv, np.float32)), _p(q), _p(s), n, K,
                          int(neg_zero))
    return q, s


def mxfp4_gemm(aq, a_s, wq, w_s, epi=0, out=None):
    """-> (out (bf16 bits or fp32), float64 sums [M, N])."""
    M, N, K = aq.shape[0], wq.shape[0], aq.shape[1] * 2
    dt = np.uint16 if epi == 0 else np.float32
    o = np.zeros((M, N), dt) if out is None else np.array(out, dtype=dt, copy=True, order="C")
    o64 = np.zeros((M, N), np.float64)
    lib().orc_mxfp4_gemm(_p(_c(aq, np.uint8)), _p(_c(a_s, np.uint8)), _p(_c(wq, np.uint8)), _p(_c(w_s, np.uint8)),
                         _p(o), ctypes.c_long(N), _p(o64), M, N, K, epi)
    return o, o64


def fp32_linear(x, w):
    M, K = x.shape
    N = w.shape[0]
    o = np.zeros((M, N), np.float32)
    lib().orc_fp32_linear(_p(_c(x, np.float32)), _p(_c(w, np.float32)), _p(o), M, N, K)
    return o
