"""The CPU oracle against the reference's own GPU kernels.

tests/golden/gpu_ref.npz holds what the reference's unmodified Triton kernels produced on a B200 for the seeded inputs
of tests/golden/gpu_cases.py (recorded by tests/golden/make_golden_gpu.py).  It pins the half of oracle.c that the
reference implements only as GPU code: the W8A8 GEMM and its epilogues (the reference's own test is bit-equality with
this Triton kernel, tests/test_cuda_gemm.py:56,89-90,219), fold, the per-token quantizers and the fused producers.

Exact integer work and the explicitly rounded epilogues (mul_rn / add_rn) must match bit for bit.  The quantizers use
Triton's `/`, which is not a correctly rounded division: the number of int8 values that differ from the IEEE contract
is counted and printed, never assumed, and each must differ by one step.  Producers whose sums or exponentials have no
defined order are compared within one int8 step."""
import os
import sys

import numpy as np
import pytest

import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import gpu_cases as C  # noqa: E402

PATH = os.path.join(HERE, "golden", "gpu_ref.npz")
pytestmark = pytest.mark.skipif(not os.path.exists(PATH), reason="gpu_ref.npz has not been recorded")


@pytest.fixture(scope="module")
def ref():
    return np.load(PATH)


def has(ref, key):
    if key not in ref.files:
        pytest.skip(f"{key} was not recorded (the reference kernel did not run)")
    return ref[key]


def ulp_report(what, got, want):
    """Scales: the reference divides with Triton's `/` (div.full.f32, not correctly rounded); the oracle's contract is the
    IEEE quotient.  Count the scales that differ and require them to be neighbours."""
    d = np.abs(got.view(np.uint32).astype(np.int64) - want.view(np.uint32).astype(np.int64))
    print(f"{what}: {int((d != 0).sum())} of {d.size} scales differ from the reference kernel's, by at most {d.max()} ulp")
    assert d.max() <= 2, (what, d.max())


def step_report(what, got, want):
    """Count of int8 values that differ, all of which must differ by exactly one step."""
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    n = int((d != 0).sum())
    print(f"{what}: {n} of {d.size} int8 values differ from the reference kernel ({n / d.size:.2e}), max step {d.max()}")
    assert d.max() <= 1, (what, d.max())
    return n / d.size


@pytest.mark.parametrize("name", list(C.GEMM_CASES))
def test_gemm_bits(ref, name):
    i = C.gemm_inputs(name)
    a, a_s, w, w_s = (i[k].numpy() for k in ("a", "a_s", "w", "w_s"))
    for epi in i["epis"]:
        want = has(ref, f"gemm/{name}/epi{epi}")
        got = oracle.w8a8_gemm(a, a_s, w, w_s, i["gk"], epi, i["live"], out=i["base"].numpy() if epi == 1 else None)
        if epi == 1:
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (name, epi)
        else:
            assert np.array_equal(got, want), (name, epi, np.argwhere(got != want)[:3])


def test_fold_bits(ref):
    i = C.fold_inputs()
    got = oracle.fold(i["h"].numpy(), i["parts"].numpy(), i["a_s"].numpy(), i["w_s"].numpy(), i["live"])
    assert np.array_equal(got.view(np.uint32), has(ref, "fold/h").view(np.uint32))


@pytest.mark.parametrize("name", list(C.ROWS_CASES))
def test_rows_q8(ref, name):
    i = C.rows_inputs(name)
    q, s = oracle.quant_rows(C.bits(i["x"]), None, None if i["inv"] is None else i["inv"].numpy(), i["live"])
    live = i["live"]
    ulp_report(f"rows_q8 {name}", s.reshape(-1)[:live], has(ref, f"rows/{name}/s")[:live])
    frac = step_report(f"rows_q8 {name}", q[:live], has(ref, f"rows/{name}/q")[:live])
    assert frac < 1e-3


def test_quant_rows_groups(ref):
    i = C.groups_inputs()
    q, s = oracle.quant_rows(C.bits(i["x"]), i["gk"])
    ulp_report("quant_rows gk=32", s, has(ref, "groups/s"))
    assert step_report("quant_rows gk=32", q, has(ref, "groups/q")) < 1e-3


@pytest.mark.parametrize("name", list(C.SWIGLU_CASES))
def test_swiglu_q8(ref, name):
    i = C.swiglu_inputs(name)
    live = i["live"]
    q, s = oracle.swiglu_q8(C.bits(i["gu"]), None if i["inv"] is None else i["inv"].numpy(), live)
    assert np.allclose(s[:live], has(ref, f"swiglu/{name}/s")[:live], rtol=1e-5, atol=0)
    step_report(f"swiglu_q8 {name}", q[:live], has(ref, f"swiglu/{name}/q")[:live])


@pytest.mark.parametrize("name", list(C.NORM_CASES))
def test_norm_q8(ref, name):
    i = C.norm_inputs(name)
    live = i["live"]
    h = i["h"].numpy().copy()
    kw = {}
    if i["parts"] is not None:
        kw = dict(parts=i["parts"].numpy(), psa=i["psa"].numpy(), psw=i["psw"].numpy())
    q, s = oracle.norm_q8(h, i["w"].numpy(), C.EPS, rows=None if i["rows"] is None else i["rows"].numpy(), live=live, **kw)
    assert np.allclose(s[:live], has(ref, f"norm/{name}/s")[:live], rtol=1e-5, atol=0)
    step_report(f"norm_q8 {name}", q[:live], has(ref, f"norm/{name}/q")[:live])
    if i["parts"] is not None:                           # the deferred add finished inside the norm: exact roundings
        assert np.array_equal(h[:live].view(np.uint32), has(ref, f"norm/{name}/h")[:live].view(np.uint32))


def test_gated_norm_q8(ref):
    i = C.gated_inputs()
    live = i["live"]
    q, s = oracle.gated_norm_q8(i["o"].numpy(), C.bits(i["proj"]), i["z_off"], i["w"].numpy(), i["inv"].numpy(), i["HV"],
                                i["D"], C.EPS, live)
    assert np.allclose(s[:live], has(ref, "gated/s")[:live], rtol=1e-5, atol=0)
    step_report("gated_norm_q8", q[:live], has(ref, "gated/q")[:live])


def test_head(ref):
    i = C.head_inputs()
    live = i["live"]
    q, s = oracle.head_quant(i["h"].numpy(), i["w"].numpy(), C.EPS, live)
    assert np.allclose(s[:live], has(ref, "head/s")[:live], rtol=1e-5, atol=0)
    step_report("head_quant", q[:live], has(ref, "head/q")[:live])
    # the head GEMM on the reference's own int8 rows: the reference writes `acc += (ai * sa) * sw` without explicit
    # roundings and its compiler fuses the second multiply with the add; the oracle's epi 4 states exactly that
    rq, rs = has(ref, "head/q"), has(ref, "head/s")
    got = oracle.w8a8_gemm(rq[:live], rs[:live], i["wq"].numpy(), i["wd"].float().numpy(), 32, 4, live)
    assert np.array_equal(got.view(np.uint32), has(ref, "head/logits")[:live].view(np.uint32))


@pytest.mark.parametrize("name", list(C.SWIGLU_EPI_CASES))
def test_swiglu_epilogue(ref, name):
    i = C.swiglu_epi_inputs(name)
    import torch
    FF, BN, live = i["FF"], i["BN"], i["live"]
    h = BN // 2

    def inter(g, u):
        return torch.stack([g.view(FF // h, h, -1), u.view(FF // h, h, -1)], 1).reshape(2 * FF, -1).contiguous()
    w = inter(i["gate"], i["up"]).numpy()
    ws = inter(i["gate_s"].view(FF, 1), i["up_s"].view(FF, 1)).view(-1).numpy()
    q, s = oracle.w8a8_swiglu_epi(i["a"].numpy(), i["a_s"].numpy(), w, ws, BN, live)
    assert np.allclose(s[:live], has(ref, f"epi2/{name}/s")[:live], rtol=1e-5, atol=0)
    step_report(f"gemm epi 2 {name}", q[:live], has(ref, f"epi2/{name}/q")[:live])


def test_mxfp4(ref):
    i = C.mxfp4_inputs()
    q, s = oracle.mxfp4_quant(C.bits(i["x"]))
    assert np.array_equal(q, has(ref, "mxfp4/aq")) and np.array_equal(s, has(ref, "mxfp4/as"))
    out, sums = oracle.mxfp4_gemm(has(ref, "mxfp4/aq"), has(ref, "mxfp4/as"), has(ref, "mxfp4/wq"), has(ref, "mxfp4/ws"))
    want = oracle.bf16_to_f32(has(ref, "mxfp4/out_bf16")).astype(np.float64)
    err = np.linalg.norm(want - sums) / np.linalg.norm(sums)
    print(f"reference tl.dot_scaled GEMM vs the float64 dequantized product: rel-Frobenius {err:.2e}")
    assert err < 2e-3                                    # the reference's own bound (tests/test_mxfp4.py:77)
    add = has(ref, "mxfp4/out_add").astype(np.float64) - i["base"].numpy().astype(np.float64)
    assert np.linalg.norm(add - sums) / np.linalg.norm(sums) < 1e-4
