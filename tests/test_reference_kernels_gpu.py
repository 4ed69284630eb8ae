"""This library's CUDA kernels against what the reference's own Triton kernels produced on a B200 for the same seeded
inputs (tests/golden/gpu_ref.npz, recorded by tests/golden/make_golden_gpu.py): no oracle in between.  The bars are the
reference's: GEMM outputs and the fold bit for bit (tests/test_cuda_gemm.py:56,89-90,219), quantizer scales bit for bit
and int8 values equal except where Triton's approximate division lands on the other side of a rounding boundary (the
count is printed), fused producers within one int8 step, MXFP4 within 1e-3 relative Frobenius error."""
import os
import sys
import types

import numpy as np
import pytest
import torch

from prism_b200 import decode, mxfp4, quant, w8a8
from util import n_rows

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import gpu_cases as C  # noqa: E402

PATH = os.path.join(HERE, "golden", "gpu_ref.npz")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(PATH), reason="gpu_ref.npz has not been recorded")]


@pytest.fixture(scope="module")
def ref():
    return np.load(PATH)


def has(ref, key):
    if key not in ref.files:
        pytest.skip(f"{key} was not recorded")
    return ref[key]


def ulps(what, got, want):
    d = np.abs(got.view(np.uint32).astype(np.int64) - want.view(np.uint32).astype(np.int64))
    print(f"{what}: {int((d != 0).sum())} of {d.size} scales differ from the reference kernel's, by at most {d.max()} ulp")
    assert d.max() <= 2, what


def steps(what, got, want, limit=None):
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    frac = float((d != 0).mean())
    print(f"{what}: {int((d != 0).sum())} of {d.size} int8 values differ from the reference kernel's, max step {d.max()}")
    assert d.max() <= 1, what
    if limit is not None:
        assert frac < limit, (what, frac)


@pytest.mark.parametrize("name", list(C.GEMM_CASES))
def test_gemm(dev, ref, name):
    i = C.gemm_inputs(name)
    M, N, gk, live = i["M"], i["N"], i["gk"], i["live"]
    a, a_s, w, w_s = (i[k].to(dev) for k in ("a", "a_s", "w", "w_s"))
    nr = n_rows(live, dev)
    for epi in i["epis"]:
        want = has(ref, f"gemm/{name}/epi{epi}")
        if epi == 0:
            out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
            w8a8.gemm(a, a_s, w, w_s, out, nr, gk, epi=0)
            assert np.array_equal(C.bits(out), want), (name, epi)
        elif epi == 1:
            out = i["base"].to(dev)
            w8a8.gemm(a, a_s, w, w_s, out, nr, gk, epi=1)
            assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32)), (name, epi)
        else:
            slots = torch.zeros(1, M, N, dtype=torch.int32, device=dev)
            assert w8a8.gemm_i32(a, a_s.view(-1), w, w_s.view(-1), slots, nr, max_split=1) == 1
            assert np.array_equal(slots[0].cpu().numpy(), want), (name, epi)


def test_fold(dev, ref):
    i = C.fold_inputs()
    h = i["h"].to(dev)
    quant.fold(h, i["parts"].to(dev), w8a8.Deferred(i["S"], i["a_s"].to(dev), i["w_s"].to(dev)), n_rows(i["live"], dev),
               i["rows"])
    assert np.array_equal(h.cpu().numpy().view(np.uint32), has(ref, "fold/h").view(np.uint32))


@pytest.mark.parametrize("name", list(C.ROWS_CASES))
def test_rows_q8(dev, ref, name):
    i = C.rows_inputs(name)
    T, K, live = i["T"], i["K"], i["live"]
    q = torch.zeros(T, K, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    quant.rows_q8(i["x"].to(dev), None if i["inv"] is None else i["inv"].to(dev), q, s, n_rows(live, dev), T)
    ulps(f"rows_q8 {name}", s.cpu().numpy()[:live], has(ref, f"rows/{name}/s")[:live])
    steps(f"rows_q8 {name}", q.cpu().numpy()[:live], has(ref, f"rows/{name}/q")[:live], 1e-3)


def test_quant_rows_groups(dev, ref):
    i = C.groups_inputs()
    q, s = w8a8.quant_rows(i["x"].to(dev), i["gk"])
    ulps("quant_rows", s.cpu().numpy(), has(ref, "groups/s"))
    steps("quant_rows", q.cpu().numpy(), has(ref, "groups/q"), 1e-3)


@pytest.mark.parametrize("name", list(C.SWIGLU_CASES))
def test_swiglu_q8(dev, ref, name):
    i = C.swiglu_inputs(name)
    T, FF, live = i["T"], i["FF"], i["live"]
    q = torch.zeros(T, FF, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    quant.swiglu_q8(i["gu"].to(dev), None if i["inv"] is None else i["inv"].to(dev), q, s, n_rows(live, dev), T)
    assert np.allclose(s.cpu().numpy()[:live], has(ref, f"swiglu/{name}/s")[:live], rtol=1e-5, atol=0)
    steps(f"swiglu_q8 {name}", q.cpu().numpy()[:live], has(ref, f"swiglu/{name}/q")[:live], 0.02)


@pytest.mark.parametrize("name", list(C.NORM_CASES))
def test_norm_q8(dev, ref, name):
    i = C.norm_inputs(name)
    T, HID, live = i["T"], i["HID"], i["live"]
    h = i["h"].to(dev)
    q = torch.zeros(T, HID, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    pend = parts = None
    if i["parts"] is not None:
        parts = i["parts"].to(dev)
        pend = w8a8.Deferred(parts.shape[0], i["psa"].to(dev), i["psw"].to(dev))
    quant.norm_q8(h, i["w"].to(dev), q, s, n_rows(live, dev), T, C.EPS,
                  rows=None if i["rows"] is None else i["rows"].to(dev), parts=parts, pending=pend)
    assert np.allclose(s.cpu().numpy()[:live], has(ref, f"norm/{name}/s")[:live], rtol=1e-5, atol=0)
    steps(f"norm_q8 {name}", q.cpu().numpy()[:live], has(ref, f"norm/{name}/q")[:live], 0.02)
    if i["parts"] is not None:
        assert np.array_equal(h.cpu().numpy()[:live].view(np.uint32), has(ref, f"norm/{name}/h")[:live].view(np.uint32))


def test_gated_norm_q8(dev, ref):
    i = C.gated_inputs()
    T, HV, D, live = i["T"], i["HV"], i["D"], i["live"]
    cfg = types.SimpleNamespace(eps=C.EPS, v_heads=HV, gdn_dim=D)
    q = torch.zeros(T, HV * D, dtype=torch.int8, device=dev)
    s = torch.zeros(T, device=dev)
    quant.gated_norm_q8(i["o"].to(dev), i["proj"].to(dev), i["z_off"], i["w"].to(dev), i["inv"].to(dev), q, s,
                        n_rows(live, dev), T, cfg)
    assert np.allclose(s.cpu().numpy()[:live], has(ref, "gated/s")[:live], rtol=1e-5, atol=0)
    steps("gated_norm_q8", q.cpu().numpy()[:live], has(ref, "gated/q")[:live], 0.02)


def test_head(dev, ref):
    i = C.head_inputs()
    B, HID, N, live = i["B"], i["HID"], i["N"], i["live"]
    q = torch.zeros(B, HID, dtype=torch.int8, device=dev)
    s = torch.zeros(B, HID // 32, device=dev)
    decode.head_quant(i["h"].to(dev), i["w"].to(dev), q, s, n_rows(live, dev), B, C.EPS)
    assert np.allclose(s.cpu().numpy()[:live], has(ref, "head/s")[:live], rtol=1e-5, atol=0)
    steps("head_quant", q.cpu().numpy()[:live], has(ref, "head/q")[:live], 0.02)
    # the head GEMM on the reference's own int8 rows and scales
    rq = torch.from_numpy(has(ref, "head/q")).to(dev)
    rs = torch.from_numpy(has(ref, "head/s")).to(dev)
    logits = torch.zeros(B, N, device=dev)
    decode.head_q8(rq, rs, i["wq"].to(dev), i["wd"].t().contiguous().to(dev), logits, n_rows(live, dev), B)
    got, want = logits.cpu().numpy()[:live], has(ref, "head/logits")[:live]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))       # bit for bit


@pytest.mark.parametrize("name", list(C.SWIGLU_EPI_CASES))
def test_gemm_swiglu_epilogue(dev, ref, name):
    i = C.swiglu_epi_inputs(name)
    M, FF, K, BN, live = i["M"], i["FF"], i["K"], i["BN"], i["live"]
    w = w8a8.interleave_gate_up(i["gate"], i["up"], BN).to(dev)
    ws = w8a8.interleave_gate_up(i["gate_s"].view(FF, 1), i["up_s"].view(FF, 1), BN).view(-1).to(dev)
    q = torch.zeros(M, FF, dtype=torch.int8, device=dev)
    s = torch.zeros(M, 2 * FF // BN, device=dev)
    w8a8.gemm(i["a"].to(dev), i["a_s"].to(dev), w, ws, q, n_rows(live, dev), K, epi=2, outs=s, cfg=(64, BN, 64, 8, 8, 3, 1))
    assert np.allclose(s.cpu().numpy()[:live], has(ref, f"epi2/{name}/s")[:live], rtol=1e-5, atol=0)
    steps(f"gemm epi 2 {name}", q.cpu().numpy()[:live], has(ref, f"epi2/{name}/q")[:live], 0.02)


def test_mxfp4(dev, ref):
    i = C.mxfp4_inputs()
    M, N, K = i["M"], i["N"], i["K"]
    q = torch.zeros(M, K // 2, dtype=torch.uint8, device=dev)
    s = torch.zeros(M, K // 32, dtype=torch.uint8, device=dev)
    mxfp4.quantize_act(i["x"].to(dev), q, s)
    assert np.array_equal(q.cpu().numpy(), has(ref, "mxfp4/aq")) and np.array_equal(s.cpu().numpy(), has(ref, "mxfp4/as"))
    w = mxfp4.MX4(torch.from_numpy(has(ref, "mxfp4/wq")).to(dev), torch.from_numpy(has(ref, "mxfp4/ws")).to(dev), N, K)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    mxfp4.gemm(q, s, w, out, M, epi=0)
    want = torch.from_numpy(has(ref, "mxfp4/out_bf16").view(np.int16)).view(torch.bfloat16).double().numpy()
    got = out.double().cpu().numpy()
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    same = (C.bits(out) == has(ref, "mxfp4/out_bf16")).mean()
    print(f"mxfp4 gemm vs the reference's tl.dot_scaled kernel: rel-Frobenius {err:.2e}, {same:.4f} of bf16 outputs bit-equal")
    assert err < 1e-3
    res = i["base"].to(dev)
    mxfp4.gemm(q, s, w, res, M, epi=1)
    want1 = has(ref, "mxfp4/out_add").astype(np.float64) - i["base"].numpy().astype(np.float64)
    got1 = res.double().cpu().numpy() - i["base"].numpy().astype(np.float64)
    assert np.linalg.norm(got1 - want1) / np.linalg.norm(want1) < 1e-4


def test_quantizers_with_the_reference_division(dev, ref):
    """The default quantizers divide by IEEE rules (the contract the oracle states); the reference's Triton `/` is the
    approximate full-range division.  With PRISM_B200_QUANT_DIV=full (read when the library first quantizes, hence a
    child process) this library divides the same way, and then scales AND int8 values must equal the reference
    kernel's bit for bit: the only difference between the two builds of the quantizer is the division."""
    import subprocess
    if os.environ.get("PRISM_B200_QUANT_DIV") != "full":
        env = dict(os.environ, PRISM_B200_QUANT_DIV="full")
        r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-s", "-m", "gpu", "-p", "no:cacheprovider", __file__,
                            "-k", "test_quantizers_with_the_reference_division"], env=env, capture_output=True, text=True)
        print(r.stdout[-1500:])
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
        return
    for name in C.ROWS_CASES:
        i = C.rows_inputs(name)
        T, K, live = i["T"], i["K"], i["live"]
        q = torch.zeros(T, K, dtype=torch.int8, device=dev)
        s = torch.zeros(T, device=dev)
        quant.rows_q8(i["x"].to(dev), None if i["inv"] is None else i["inv"].to(dev), q, s, n_rows(live, dev), T)
        assert np.array_equal(s.cpu().numpy()[:live].view(np.uint32), has(ref, f"rows/{name}/s")[:live].view(np.uint32)), name
        assert np.array_equal(q.cpu().numpy()[:live], has(ref, f"rows/{name}/q")[:live]), name
    i = C.groups_inputs()
    q, s = w8a8.quant_rows(i["x"].to(dev), i["gk"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), has(ref, "groups/s").view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), has(ref, "groups/q"))
