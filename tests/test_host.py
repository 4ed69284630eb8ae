"""Host-side logic on the CPU: weight containers and encoders against gguf-py and the golden vectors, weight
preparation, sharding indices, the C-ABI library's exported symbols (no kernel is launched)."""
import ctypes
import os
import re
import types

import numpy as np
import pytest
import torch

from prism_b200 import _lib, gguf_weights as GW, synth, tp, w8a8

G = os.path.join(os.path.dirname(__file__), "golden")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load(name):
    return np.load(os.path.join(G, name))


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "prism_b200.h")).read()
    declared = set(re.findall(r"\b(pb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/prism_b200.h but not exported"
    assert declared == set(_lib.declared_symbols())
    assert lib.pb_version() >= 1
    assert b"ok" == lib.pb_status_string(0)


def test_operators_refuse_cpu_tensors(lib):
    a = torch.zeros(4, 64, dtype=torch.int8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        w8a8.gemm(a, torch.ones(4), a, torch.ones(4), torch.zeros(4, 4, dtype=torch.bfloat16),
                  torch.tensor([4], dtype=torch.int32), 64)


def test_argument_checks_without_gpu(lib):
    """Bad arguments are refused before any CUDA call."""
    assert lib.pb_w8a8_gemm(None, None, None, None, None, 0, None, 1, 1, 16, 16, 0, 1, 0, None, 0, None, 0, 0, None) == 1
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.pb_w8a8_gemm(p16, p16, p16, p16, p16, 8, p16, 4, 8, 24, 24, 0, 1, 0, None, 0, None, 0, 0, None) == 2  # K % 16
    assert lib.pb_w8a8_gemm(p16 + 1, p16, p16, p16, p16, 8, p16, 4, 8, 32, 32, 0, 1, 0, None, 0, None, 0, 0, None) == 1
    assert lib.pb_quant_rows(p16, 0, 32, None, p16, p16, p16, 4, 64, 64, 1, None, None) == 1   # mode 1 without amax
    assert lib.pb_w8a8_workspace_bytes(16, 5120, 4) == 4 * 40 * 16 * 128 * 4
    assert lib.pb_w8a8_counters(64, 7168) == 56
    # row blocks of the scattered int32 output: whole tiles, at most eight, covering every row
    blocks = (ctypes.c_void_p * 8)(*([p16] * 8))
    assert lib.pb_w8a8_gemm_scatter(p16, p16, blocks, 2, 100, 64, p16, 200, 64, 128, None) == 2      # block rows % 128
    assert lib.pb_w8a8_gemm_scatter(p16, p16, blocks, 9, 128, 64, p16, 256, 64, 128, None) == 1      # more than 8 blocks
    assert lib.pb_w8a8_gemm_scatter(p16, p16, blocks, 2, 128, 64, p16, 512, 64, 128, None) == 1      # rows not covered
    assert lib.pb_w8a8_gemm_scatter(p16, p16, blocks, 1, 128, 64, p16, 64, 64, 128, None) == 2       # few rows
    # MXFP4: split needs its workspace; the CUDA-core kernel takes up to four rows
    assert lib.pb_mxfp4_gemm_split(p16, p16, p16, p16, p16, 128, 16, 128, 2048, 0, 2, None, 0, None, 0, None) == 1
    assert lib.pb_mxfp4_workspace_bytes(16, 5120, 3) == 40 * 3 * 128 * 128 * 4 and lib.pb_mxfp4_counters(16, 5120) == 40
    assert lib.pb_mxfp4_gemv(p16, p16, p16, p16, p16, 128, 5, 128, 256, 0, None) == 2
    assert lib.pb_mxfp4_gemv(p16, p16, p16, p16, p16, 128, 1, 128, 128, 0, None) == 2                # K % 256


def test_split_rules_of_the_other_formats():
    from prism_b200 import mxfp4, w4a8
    # few-rows W4A8: time goes as waves / slices; Q6_K's 80 tiles of the down projection take 7 slices (4 waves)
    assert w4a8.pick_split(8, 5120, 5120, 128) == 3 and w4a8.pick_split(8, 34816, 5120, 128) == 1
    assert w4a8.pick_split(8, 5120, 17408, 64) == 7 and w4a8.pick_split(17, 5120, 17408, 64) == 1
    # MXFP4: only where one row tile's tiles leave most SMs idle
    assert mxfp4.pick_split(16, 5120, 5120) == 3 and mxfp4.pick_split(16, 34816, 5120) == 1
    assert mxfp4.pick_split(300, 5120, 5120) == 1 and mxfp4.pick_split(1, 5120, 512) == 1


def test_split_rule():
    assert w8a8.effective_split(256, 4) == 2 and w8a8.effective_split(5120, 7) == 7
    assert w8a8.effective_split(17408, 8) == 8 and w8a8.effective_split(640, 4) == 3   # 5 blocks: 2 + 2 + 1
    assert w8a8.pick_split(16, 5120, 5120) == 7 and w8a8.pick_split(16, 34816, 5120) == 1
    assert w8a8.pick_split(8192, 5120, 5120) == 1


def test_q8_and_weight_from_q8_match_reference():
    g = load("w8a8.npz")
    q8 = GW.Q8(torch.from_numpy(g["qs"]), torch.from_numpy(g["d"]))
    assert np.array_equal(q8.dequant().numpy(), g["dequant"])
    sm = torch.from_numpy(g["smooth"])
    for gk, s, tag in ((32, None, "gk32"), (64, None, "gk64"), (256, None, "gk256"), (256, sm, "gk256s"),
                       (32, sm, "gk32s")):
        q, sc = w8a8.weight_from_q8(q8, gk, s)
        assert np.array_equal(q.numpy(), g[f"q_{tag}"]) and np.array_equal(sc.numpy(), g[f"s_{tag}"]), tag
    gu = w8a8.interleave_gate_up(torch.from_numpy(g["gate"]), torch.from_numpy(g["up"]), 16)
    assert np.array_equal(gu.numpy(), g["gu16"])


def test_kquant_dequant_matches_reference_and_gguf_py():
    g = load("kquant.npz")
    from gguf.constants import GGMLQuantizationType as T
    from gguf.quants import dequantize
    for tag, typ, gt in (("4", GW.GGML_Q4_K, T.Q4_K), ("6", GW.GGML_Q6_K, T.Q6_K)):
        kq = GW.KQuant(torch.from_numpy(g[f"raw{tag}"]), typ, 512)
        got = kq.dequant().numpy()
        assert np.array_equal(got, g[f"deq{tag}"])
        assert np.array_equal(got, dequantize(g[f"raw{tag}"].reshape(24, -1), gt).reshape(24, 512))
        q8 = kq.as_q8()
        assert np.array_equal(q8.qs.numpy(), g[f"q8_{tag}_qs"]) and np.array_equal(q8.d.numpy(), g[f"q8_{tag}_d"])
    sc, mn = GW.scale_min_k4(torch.from_numpy(g["raw4"]).reshape(-1, 144)[:, 4:16])
    assert np.array_equal(sc.numpy(), g["sc"].astype(np.int32)) and np.array_equal(mn.numpy(), g["mn"].astype(np.int32))


def test_encoders_are_valid_blocks():
    """Seeded inputs: Q8_0 byte-for-byte as gguf-py quantizes; Q4_K / Q6_K blocks dequantize identically under gguf-py
    and stay close to the source weights; Q5_K dequantizes as gguf-py on random bytes."""
    from gguf.constants import GGMLQuantizationType as T
    from gguf.quants import dequantize, quantize
    w = synth.weights(32, 1024, 5)
    q8 = synth.q8_0(w)
    ref = quantize(w.numpy(), T.Q8_0).reshape(32, 32, 34)
    assert np.array_equal(ref[..., 2:].copy().view(np.int8).reshape(32, 1024), q8.qs.numpy())
    assert np.array_equal(ref[..., :2].copy().view(np.float16).reshape(32, 32), q8.d.numpy())
    assert np.array_equal(GW.Q8.from_blocks(torch.from_numpy(ref.reshape(-1)), 32, 1024).qs.numpy(), q8.qs.numpy())
    for enc, gt, tol in ((synth.q4_k, T.Q4_K, 0.12), (synth.q6_k, T.Q6_K, 0.04)):
        kq = enc(w)
        d = kq.dequant().numpy()
        assert np.array_equal(d, dequantize(kq.raw.numpy().reshape(32, -1), gt).reshape(32, 1024))
        assert np.linalg.norm(d - w.numpy()) / np.linalg.norm(w.numpy()) < tol
    raw = torch.randint(0, 256, (8, 2, 176), dtype=torch.uint8, generator=torch.Generator().manual_seed(0))
    raw[..., 1] = 0x2c                      # keep the fp16 d / dmin finite
    raw[..., 3] = 0x2c
    k5 = GW.KQuant(raw, GW.GGML_Q5_K, 512)
    assert np.array_equal(k5.dequant().numpy(), dequantize(raw.numpy().reshape(8, -1), T.Q5_K).reshape(8, 512))


def test_shard_index_matches_reference():
    g = load("tp.npz")
    cfg = types.SimpleNamespace(n_head=20, n_kv_head=4, head_dim=128, k_heads=16, v_heads=48, gdn_dim=128, ffn=17408)
    for n in (2, 4):
        for r in range(n):
            for k, v in tp.shard_index(cfg, n, r).items():
                assert np.array_equal(v.numpy(), g[f"n{n}_r{r}_{k}"]), (n, r, k)


def test_linear_shards_partition():
    for n in (1, 2, 4, 8):
        seen = {k: [] for k in ("qkv", "o", "gu", "down")}
        for r in range(n):
            for k, v in tp.linear_shards(5120, 1024, 17408, n, r).items():
                seen[k].append(v)
        assert torch.equal(torch.cat(seen["qkv"]).sort().values, torch.arange(7168))
        assert torch.equal(torch.cat(seen["o"]), torch.arange(5120))
        assert torch.equal(torch.cat(seen["gu"]).sort().values, torch.arange(34816))
        assert torch.equal(torch.cat(seen["down"]), torch.arange(17408))
    with pytest.raises(ValueError):
        tp.linear_shards(5120, 1024, 17408, 3, 0)
    assert tp.parts_elems(64, 5120) == 4 * 64 * 5120 and tp.parts_elems(8192, 5120) == 8192 * 5120


def test_w4a8_repack_matches_reference():
    from prism_b200 import w4a8
    g, k = load("w4a8.npz"), load("kquant.npz")
    w = w4a8.repack(GW.KQuant(torch.from_numpy(k["raw4"]), GW.GGML_Q4_K, 512))
    assert w.kind == "q4k" and (w.n, w.k) == (24, 512)
    for f in ("q", "sc", "mn", "d", "dm"):
        assert np.array_equal(getattr(w, f).numpy(), g[f + "4"]), f
    w6 = w4a8.repack(GW.KQuant(torch.from_numpy(k["raw6"]), GW.GGML_Q6_K, 512))
    for f in ("q", "sc", "d"):
        assert np.array_equal(getattr(w6, f).numpy(), g[f + "6"]), f
    assert w6.mn is None and w6.dm is None
    both = w4a8.concat([w, w])
    assert both.n == 48 and both.sc.shape == (2, 48, 8) and both.q.shape == (48, 256)
    part = both.rows(10, 30)
    assert part.n == 20 and np.array_equal(part.d.numpy(), np.concatenate([g["d4"], g["d4"]], 1)[:, 10:30])
    with pytest.raises(ValueError):
        w4a8.concat([w, w6])


def test_mxfp4_pack_matches_reference():
    from prism_b200 import mxfp4
    g = load("mxfp4.npz")
    w = torch.from_numpy(g["w"])
    for mode in ("max", "mse"):
        m = mxfp4.pack(w, mode)
        assert np.array_equal(m.q.numpy(), g[f"q_{mode}"]) and np.array_equal(m.s.numpy(), g[f"s_{mode}"]), mode
        assert np.array_equal(mxfp4.dequant_packed(m.q, m.s).numpy(), g[f"deq_{mode}"])
    m = mxfp4.pack(torch.from_numpy(g["grid"]))                   # tests/test_mxfp4.py:34-38: exact-grid values survive
    assert np.array_equal(m.q.numpy(), g["grid_q"]) and np.array_equal(m.s.numpy(), g["grid_s"])
    assert float((mxfp4.dequant_packed(m.q, m.s) - torch.from_numpy(g["grid"])).abs().max()) < 1e-6
    assert mxfp4.MX4(m.q, m.s, 1, 32).rows(0, 1).shape == (1, 32)
