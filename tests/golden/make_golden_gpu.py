"""Records the outputs of the reference's own GPU kernels (its Triton kernels, run unmodified on a B200) for the seeded
inputs of gpu_cases.py -> gpu_ref.npz.  This pins the half of the CPU oracle that exists in the reference only as
Triton code: the W8A8 GEMM with its epilogues (one scale group, per-32 / per-64 / per-128 groups, the fused SwiGLU
epilogue), the per-token quantizers (rows_q8, swiglu_q8, norm_q8 with and without a deferred add, gated_norm_q8,
quant_rows, head_quant), fold, the vocabulary head GEMM and the MXFP4 quantizer + tl.dot_scaled GEMM.

Run on a machine with a GPU and a checkout of the reference (never part of a test run):

    python tests/golden/make_golden_gpu.py <dir that holds the startlux_prism package> <output.npz>

Only tensor-parallel modes 0 are run: the reference's cross-rank spins (mode 3, _tp_sync) have no bound and are not
touched.  Every case is wrapped: a kernel that fails to compile or run is reported and left out of the file."""
import os
import sys
import traceback
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if len(sys.argv) < 3:
    raise SystemExit("usage: make_golden_gpu.py <dir with startlux_prism/> <output.npz>")
sys.path.insert(0, sys.argv[1])
sys.path.insert(0, HERE)
os.environ["STARTLUX_PRISM_GEMM"] = "triton"            # no dispatch table: the Triton kernels themselves

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton.language as tl  # noqa: E402
from triton.language import core as _tl_core  # noqa: E402

import gpu_cases as C  # noqa: E402

# The reference pins Triton 3.8, where tl.dot(a, b, acc) takes its result type from the accumulator.  Older Tritons
# (3.6 is what this image has) assert acc.dtype == out_dtype with out_dtype defaulting to float32, so the reference's
# int8 dot into an int32 accumulator (kernels/w8a8.py:58,70) fails to compile there.  This shim changes nothing but that
# default - out_dtype = the accumulator's type when one is given - and leaves the reference's source untouched.
_dot = tl.dot


@_tl_core.builtin
def _dot_typed_by_acc(input, other, acc=None, input_precision=None, allow_tf32=None, max_num_imprecise_acc=None,
                      out_dtype=None, _semantic=None):
    if out_dtype is None:
        out_dtype = acc.dtype if acc is not None else tl.float32
    return _dot(input, other, acc, input_precision, allow_tf32, max_num_imprecise_acc, out_dtype, _semantic=_semantic)


if tuple(int(x) for x in __import__("triton").__version__.split(".")[:2]) < (3, 8):
    tl.dot = _tl_core.dot = _dot_typed_by_acc
from startlux_prism.kernels import decode as RDEC  # noqa: E402
from startlux_prism.kernels import mxfp4 as RMX  # noqa: E402
from startlux_prism.kernels import quant as RQ  # noqa: E402
from startlux_prism.kernels import w8a8 as RW8  # noqa: E402

dev = torch.device("cuda", 0)
OUT, FAILED = {}, []


def keep(name, t):
    if t.dtype == torch.bfloat16:
        OUT[name] = C.bits(t)
    else:
        OUT[name] = np.ascontiguousarray(t.detach().cpu().numpy())


def case(fn):
    try:
        fn()
        torch.cuda.synchronize()
    except Exception:                                   # noqa: BLE001
        FAILED.append(fn.__name__)
        print(f"FAILED {fn.__name__}:\n{traceback.format_exc()}", flush=True)
    return fn


def nrows(v):
    return torch.tensor([v], dtype=torch.int32, device=dev)


@case
def gemms():
    for name in C.GEMM_CASES:
        i = C.gemm_inputs(name)
        M, N, K, gk, live = i["M"], i["N"], i["K"], i["gk"], i["live"]
        a, a_s, w, w_s = (i[k].to(dev) for k in ("a", "a_s", "w", "w_s"))
        for epi in i["epis"]:
            cfg = RW8.pick(M, N, K, epi if epi != 3 else 0)
            if epi == 0:
                out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
            elif epi == 1:
                out = i["base"].to(dev)
            else:
                out = torch.zeros(M, N, dtype=torch.int32, device=dev)
            RW8.gemm(a, a_s, w, w_s, out, nrows(live), gk, epi=epi, cfg=cfg)
            keep(f"gemm/{name}/epi{epi}", out)


@case
def swiglu_epilogue():
    for name in C.SWIGLU_EPI_CASES:
        i = C.swiglu_epi_inputs(name)
        M, FF, K, BN, live = i["M"], i["FF"], i["K"], i["BN"], i["live"]
        w = RW8.interleave_gate_up(i["gate"], i["up"], BN).to(dev)
        w_s = RW8.interleave_gate_up(i["gate_s"].view(FF, 1), i["up_s"].view(FF, 1), BN).view(-1, 1).contiguous().to(dev)
        out = torch.zeros(M, FF, dtype=torch.int8, device=dev)
        outs = torch.zeros(M, 2 * FF // BN, dtype=torch.float32, device=dev)
        RW8.gemm(i["a"].to(dev), i["a_s"].to(dev), w, w_s, out, nrows(live), K, epi=2, outs=outs,
                 cfg=(64, BN, 64, 8, 8, 3, 1))
        keep(f"epi2/{name}/q", out)
        keep(f"epi2/{name}/s", outs)


@case
def rows():
    for name in C.ROWS_CASES:
        i = C.rows_inputs(name)
        T, K = i["T"], i["K"]
        inv = (i["inv"] if i["inv"] is not None else torch.ones(K)).to(dev)
        q = torch.zeros(T, K, dtype=torch.int8, device=dev)
        s = torch.zeros(T, dtype=torch.float32, device=dev)
        RQ.rows_q8(i["x"].to(dev), inv, q, s, nrows(i["live"]), T)
        keep(f"rows/{name}/q", q)
        keep(f"rows/{name}/s", s)


@case
def swiglus():
    for name in C.SWIGLU_CASES:
        i = C.swiglu_inputs(name)
        T, FF = i["T"], i["FF"]
        inv = (i["inv"] if i["inv"] is not None else torch.ones(FF)).to(dev)
        q = torch.zeros(T, FF, dtype=torch.int8, device=dev)
        s = torch.zeros(T, dtype=torch.float32, device=dev)
        RQ.swiglu_q8(i["gu"].to(dev), inv, q, s, nrows(i["live"]), T)
        keep(f"swiglu/{name}/q", q)
        keep(f"swiglu/{name}/s", s)


@case
def norms():
    for name in C.NORM_CASES:
        i = C.norm_inputs(name)
        T, HID = i["T"], i["HID"]
        h = i["h"].to(dev)
        q = torch.zeros(T, HID, dtype=torch.int8, device=dev)
        s = torch.zeros(T, dtype=torch.float32, device=dev)
        pend = parts = None
        if i["parts"] is not None:
            parts = i["parts"].to(dev)
            pend = RW8.Deferred(parts.shape[0], i["psa"].to(dev), i["psw"].to(dev))
        rows_t = i["rows"].to(dev) if i["rows"] is not None else None
        RQ.norm_q8(h, i["w"].to(dev), q, s, nrows(i["live"]), T, C.EPS, rows=rows_t, parts=parts, pending=pend)
        keep(f"norm/{name}/q", q)
        keep(f"norm/{name}/s", s)
        keep(f"norm/{name}/h", h)


@case
def fold():
    i = C.fold_inputs()
    h = i["h"].to(dev)
    parts = i["parts"].to(dev)
    RQ.fold(h, parts, RW8.Deferred(i["S"], i["a_s"].to(dev), i["w_s"].to(dev)), nrows(i["live"]), i["rows"])
    keep("fold/h", h)


@case
def groups():
    i = C.groups_inputs()
    q, s = RW8.quant_rows(i["x"].to(dev), i["gk"])
    keep("groups/q", q)
    keep("groups/s", s)


@case
def gated():
    i = C.gated_inputs()
    T, HV, D = i["T"], i["HV"], i["D"]
    cfg = types.SimpleNamespace(eps=C.EPS, v_heads=HV, gdn_dim=D)
    q = torch.zeros(T, HV * D, dtype=torch.int8, device=dev)
    s = torch.zeros(T, dtype=torch.float32, device=dev)
    RQ.gated_norm_q8(i["o"].to(dev), i["proj"].to(dev), i["z_off"], i["w"].to(dev), i["inv"].to(dev), q, s,
                     nrows(i["live"]), T, cfg)
    keep("gated/q", q)
    keep("gated/s", s)


@case
def head():
    i = C.head_inputs()
    B, HID, N = i["B"], i["HID"], i["N"]
    q = torch.zeros(B, HID, dtype=torch.int8, device=dev)
    s = torch.zeros(B, HID // 32, dtype=torch.float32, device=dev)
    RDEC.head_quant(i["h"].to(dev), i["w"].to(dev), q, s, nrows(i["live"]), B, C.EPS)
    keep("head/q", q)
    keep("head/s", s)
    logits = torch.zeros(B, N, dtype=torch.float32, device=dev)
    w_s = i["wd"].t().contiguous().to(dev)              # fp16, group-major [K / 32, N]
    RDEC.head_q8(q, s, i["wq"].to(dev), w_s, logits, nrows(i["live"]), B)
    keep("head/logits", logits)


@case
def mxfp4():
    i = C.mxfp4_inputs()
    M, N, K = i["M"], i["N"], i["K"]
    q = torch.zeros(M, K // 2, dtype=torch.uint8, device=dev)
    s = torch.zeros(M, K // 32, dtype=torch.uint8, device=dev)
    RMX.quantize_act(i["x"].to(dev), q, s)
    keep("mxfp4/aq", q)
    keep("mxfp4/as", s)
    w = RMX.pack(i["w"], "max")
    wd = RMX.MX4(w.q.to(dev), w.s.to(dev), w.n, w.k)
    keep("mxfp4/wq", w.q)
    keep("mxfp4/ws", w.s)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    RMX.gemm(q, s, wd, out, M, epi=0)
    keep("mxfp4/out_bf16", out)
    res = i["base"].to(dev)
    RMX.gemm(q, s, wd, res, M, epi=1)
    keep("mxfp4/out_add", res)


if __name__ == "__main__":
    import triton
    OUT["meta/versions"] = np.array([f"torch {torch.__version__}", f"triton {triton.__version__}",
                                     torch.cuda.get_device_name(0)])
    OUT["meta/failed"] = np.array(FAILED or ["-"])
    np.savez_compressed(sys.argv[2], **OUT)
    print(f"wrote {sys.argv[2]}: {len(OUT)} arrays; failed: {FAILED or 'none'}")
    for k, v in sorted(OUT.items()):
        print(" ", k, v.shape, v.dtype)
