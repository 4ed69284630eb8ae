"""ctypes binding of libprism_b200.so (include/prism_b200.h).  Loading fails loudly when the library is missing: the
operators have no other implementation."""
import ctypes
import functools
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "libprism_b200.so")

_vp, _i, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long


class SyncStruct(ctypes.Structure):
    """pb_sync of include/prism_b200.h."""
    _fields_ = [("epoch", ctypes.c_void_p), ("bufs", ctypes.c_void_p * 8), ("others", ctypes.c_void_p * 7),
                ("off", ctypes.c_long), ("rank", ctypes.c_int), ("world", ctypes.c_int)]


_sp = ctypes.POINTER(SyncStruct)
_SIGS = {
    "pb_version": ([], _i),
    "pb_status_string": ([_i], ctypes.c_char_p),
    "pb_last_cuda_error": ([], _i),
    "pb_device_status": ([ctypes.POINTER(_i), ctypes.POINTER(ctypes.c_uint), _i], _i),
    "pb_set_wait_limit_ns": ([ctypes.c_ulonglong], _i),
    "pb_test_drop_loads": ([_i], _i),
    "pb_w8a8_workspace_bytes": ([_i, _i, _i], _l),
    "pb_w8a8_counters": ([_i, _i], _i),
    "pb_w8a8_gemm": ([_vp, _vp, _vp, _vp, _vp, _l, _vp, _i, _i, _i, _i, _i, _i, _l, _vp, _l, _vp, _i, _i, _vp], _i),
    "pb_w8a8_gemm_swiglu": ([_vp, _vp, _vp, _vp, _vp, _l, _vp, _vp, _i, _i, _i, _i, _vp], _i),
    "pb_w8a8_gemm_scatter": ([_vp, _vp, _vp, _i, _i, _l, _vp, _i, _i, _i, _vp], _i),
    "pb_peer_alloc": ([_l, _vp, _vp], _i),
    "pb_peer_open": ([_vp, _vp], _i),
    "pb_peer_close": ([_vp], _i),
    "pb_peer_free": ([_vp], _i),
    "pb_quant_rows_exchange": ([_vp, _i, _l, _vp, _vp, _vp, _vp, _i, _i, _sp, _vp], _i),
    "pb_swiglu_q8_exchange": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _sp, _vp], _i),
    "pb_gated_norm_q8_exchange": ([_vp, _vp, _l, _l, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, ctypes.c_float, _sp, _vp], _i),
    "pb_fold_sync": ([_vp, _l, _vp, _l, _i, _vp, _vp, _vp, _i, _i, _sp, _vp], _i),
    "pb_norm_q8_sync": ([_vp, _vp, _vp, _vp, _vp, _i, _i, ctypes.c_float, _vp, _l, _i, _vp, _vp, _sp, _vp], _i),
    "pb_l2_prefetch": ([_vp, _vp, _i, _i, _vp], _i),
    "pb_fold": ([_vp, _l, _vp, _l, _i, _vp, _vp, _vp, _i, _i, _vp], _i),
    "pb_quant_rows": ([_vp, _i, _l, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp], _i),
    "pb_swiglu_q8": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp], _i),
    "pb_gated_norm_q8": ([_vp, _vp, _l, _l, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, ctypes.c_float, _i, _vp, _vp], _i),
    "pb_swiglu_g": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp], _i),
    "pb_norm_g": ([_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, ctypes.c_float, _vp], _i),
    "pb_gated_norm_g": ([_vp, _vp, _l, _l, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, ctypes.c_float, _vp], _i),
    "pb_head_quant": ([_vp, _vp, _vp, _vp, _vp, _i, _i, ctypes.c_float, _vp], _i),
    "pb_norm_q8": ([_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, ctypes.c_float, _vp, _l, _i, _vp, _vp, _vp], _i),
    "pb_quant_g": ([_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp], _i),
    "pb_mxfp4_sf_bytes": ([_i, _i], _l),
    "pb_mxfp4_prepare_sf": ([_vp, _vp, _i, _i, _vp], _i),
    "pb_mxfp4_quant": ([_vp, _i, _vp, _vp, _vp, _i, _i, _vp], _i),
    "pb_mxfp4_gemm": ([_vp, _vp, _vp, _vp, _vp, _l, _i, _i, _i, _i, _vp], _i),
    "pb_mxfp4_gemv": ([_vp, _vp, _vp, _vp, _vp, _l, _i, _i, _i, _i, _vp], _i),
    "pb_mxfp4_workspace_bytes": ([_i, _i, _i], _l),
    "pb_mxfp4_counters": ([_i, _i], _i),
    "pb_mxfp4_gemm_split": ([_vp, _vp, _vp, _vp, _vp, _l, _i, _i, _i, _i, _i, _vp, _l, _vp, _i, _vp], _i),
    "pb_w4a8_gemm": ([_vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _l, _vp, _i, _i, _i, _i, _i, _vp, _l, _vp, _i,
                      _vp], _i),
    "pb_w4a8_workspace_bytes": ([_i, _i, _i], _l),
    "pb_w4a8_counters": ([_i, _i], _i),
}
# entry points added by later sections of the header; bound when present in the built library
_OPTIONAL = {
    "pb_int8_peak_probe": ([_i, _i, _i, _vp, _vp], _i),
    "pb_mxf4_peak_probe": ([_i, _i, _vp, _vp], _i),
    "pb_set_pdl": ([_i], _i),
    "pb_push": ([_vp, _vp, _i, _l, _vp], _i),
    "pb_handshake": ([_vp, _vp], _i),
    "pb_w8a8_static_scratch_bytes": ([], _l),
    "pb_w8a8_gemm_static": ([_vp, _vp, _vp, _vp, _vp, _l, _vp, _i, _i, _i, _i, _i, _vp], _i),
}


@functools.lru_cache(None)
def lib():
    if not os.path.exists(PATH):
        raise RuntimeError(f"{PATH} is not built: run `python -m prism_b200.build` (nvcc, sm_100a).  prism_b200 has no "
                           "fallback implementation.")
    L = ctypes.CDLL(PATH)
    for name, (args, res) in {**_SIGS, **_OPTIONAL}.items():
        fn = getattr(L, name)
        fn.argtypes, fn.restype = args, res
    return L


def declared_symbols():
    return sorted({**_SIGS, **_OPTIONAL})


class PrismError(RuntimeError):
    def __init__(self, status, what):
        L = lib()
        msg = L.pb_status_string(status).decode()
        if status == 3:
            msg += f" (CUDA error {L.pb_last_cuda_error()})"
        super().__init__(f"{what}: {msg} [status {status}]")
        self.status = status


def check(status, what):
    if status:
        raise PrismError(status, what)


def ptr(t):
    return None if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("prism_b200 operators take CUDA tensors only (there is no CPU path)")


def device_status(reset=True):
    """(code, where) of the current device's status word (synchronizes)."""
    c, w = ctypes.c_int(0), ctypes.c_uint(0)
    check(lib().pb_device_status(ctypes.byref(c), ctypes.byref(w), int(reset)), "pb_device_status")
    if c.value and reset:
        # a launch that gave up may have left split-K arrival counters non-zero: later products would skip their
        # epilogue.  Every module's counters on this device start again from zero.
        from . import w8a8
        w8a8.reset_workspace()
    return c.value, w.value
