"""The GGUF reader and the loader on a small file written by gguf-py's own writer (the third-party anchor of the
format): metadata values of every kind, Q8_0 tensors quantized by gguf-py's `quantize`, Q4_K / Q6_K tensors from this
package's encoders (checked bit for bit against gguf-py's `dequantize`), F32 norms; then the conversions into the
kernels' layouts and their on-disk cache.  CPU only."""
import os

import numpy as np
import pytest
import torch

gguf_py = pytest.importorskip("gguf")

from prism_b200 import gguf as G  # noqa: E402
from prism_b200 import gguf_weights as GW  # noqa: E402
from prism_b200 import loader, mxfp4, synth, w4a8, w8a8  # noqa: E402

HID, FFN, QC, KVC = 512, 1024, 512, 256


def write_model(path, layers=2):
    from gguf import GGMLQuantizationType as T
    from gguf import GGUFWriter
    from gguf.quants import quantize
    wr = GGUFWriter(str(path), "qwen35")
    wr.add_uint32("qwen35.block_count", layers)
    wr.add_uint32("qwen35.embedding_length", HID)
    wr.add_float32("qwen35.attention.layer_norm_rms_epsilon", 1e-6)
    wr.add_bool("qwen35.attention.causal", True)
    wr.add_string("general.name", "tiny")
    wr.add_array("tokenizer.scores", [0.5, 1.5, 2.5])
    wr.add_array("tokenizer.tokens", ["a", "bc", "d"])
    truth = {}
    for i in range(layers):
        shapes = {"attn_q": (QC, HID), "attn_k": (KVC, HID), "attn_v": (KVC, HID), "attn_output": (HID, QC),
                  "ffn_gate": (FFN, HID), "ffn_up": (FFN, HID), "ffn_down": (HID, FFN)}
        for j, (name, (n, k)) in enumerate(shapes.items()):
            w = synth.weights(n, k, 100 * i + j)
            full = f"blk.{i}.{name}.weight"
            if i == 0:                                          # layer 0: Q8_0 throughout
                raw = quantize(w.numpy(), T.Q8_0)
                wr.add_tensor(full, raw, raw_dtype=T.Q8_0)
                truth[full] = ("q8", raw)
            else:                                               # layer 1: the Q4_K_M assignment
                six = name in ("attn_v", "ffn_down")
                kq = synth.q6_k(w) if six else synth.q4_k(w)
                raw = kq.raw.reshape(n, -1).numpy()
                wr.add_tensor(full, raw, raw_dtype=T.Q6_K if six else T.Q4_K)
                truth[full] = ("kq", kq)
        norm = (1.0 + 0.1 * torch.randn(HID, generator=torch.Generator().manual_seed(i))).numpy().astype(np.float32)
        wr.add_tensor(f"blk.{i}.attn_norm.weight", norm)
        truth[f"blk.{i}.attn_norm.weight"] = ("f32", norm)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    return truth


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    path = tmp_path_factory.mktemp("gguf") / "tiny.gguf"
    return path, write_model(path)


def test_reader_matches_gguf_py(model):
    path, truth = model
    f = G.GGUFFile(path)
    assert f.version == 3
    assert f.meta["general.architecture"] == "qwen35" and f.meta["qwen35.block_count"] == 2
    assert f.meta["qwen35.embedding_length"] == HID and f.meta["qwen35.attention.causal"] is True
    assert abs(f.meta["qwen35.attention.layer_norm_rms_epsilon"] - 1e-6) < 1e-12
    assert f.meta["tokenizer.scores"] == [0.5, 1.5, 2.5] and f.meta["tokenizer.tokens"] == ["a", "bc", "d"]
    # the same directory as gguf-py's reader
    rd = gguf_py.GGUFReader(str(path))
    theirs = {t.name: t for t in rd.tensors}
    assert set(theirs) == set(f.tensors)
    for name, t in f.tensors.items():
        assert tuple(int(d) for d in theirs[name].shape) == tuple(int(d) for d in t.dims), name
        assert int(theirs[name].tensor_type) == t.type and int(theirs[name].data_offset) == t.offset
        assert np.array_equal(np.asarray(theirs[name].data).reshape(-1).view(np.uint8), f.read(name)), name
    t = f.tensors["blk.0.ffn_down.weight"]
    assert t.dims == (FFN, HID) and t.shape == (HID, FFN) and t.type == G.GGML_Q8_0 and t.nbytes == HID * FFN // 32 * 34


def test_tensor_containers(model):
    from gguf.quants import dequantize
    path, truth = model
    f = G.GGUFFile(path)
    for name, (kind, ref) in truth.items():
        x = loader.tensor(f, name)
        if kind == "q8":
            assert isinstance(x, GW.Q8)
            want = dequantize(ref, gguf_py.GGMLQuantizationType.Q8_0)
            assert np.array_equal(x.dequant().numpy(), want), name
        elif kind == "kq":
            assert isinstance(x, GW.KQuant) and x.type == ref.type and torch.equal(x.raw, ref.raw)
            qt = gguf_py.GGMLQuantizationType.Q6_K if x.type == G.GGML_Q6_K else gguf_py.GGMLQuantizationType.Q4_K
            assert np.array_equal(x.dequant().numpy(), dequantize(ref.raw.reshape(ref.raw.shape[0], -1).numpy(), qt)), name
        else:
            assert x.dtype == torch.float32 and np.array_equal(x.numpy(), ref)


def test_rejects_bad_files(tmp_path):
    p = tmp_path / "x.gguf"
    p.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(ValueError, match="not a GGUF"):
        G.GGUFFile(p)
    p.write_bytes(b"GGUF" + (9).to_bytes(4, "little") + b"\0" * 32)
    with pytest.raises(ValueError, match="version 9"):
        G.GGUFFile(p)


def test_truncated_file(model, tmp_path):
    path, _ = model
    data = open(path, "rb").read()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(data[:len(data) - 1000])
    with pytest.raises(ValueError, match="truncated"):
        G.GGUFFile(cut)


def test_layouts_and_cache(model, tmp_path):
    path, truth = model
    f = G.GGUFFile(path)
    cache = loader.LayoutCache(tmp_path / "cache")
    names = [f"blk.0.{s}" for s in loader.LAYER_TENSORS["qkv"]]
    # W8A8: stacked q | k | v rows, one scale per row; equal to converting each tensor by hand
    q, s = loader.w8a8_linear(f, names, HID, cache=cache)
    assert q.shape == (QC + 2 * KVC, HID) and s.shape == (QC + 2 * KVC, 1)
    by_hand = [w8a8.weight_from_q8(loader.tensor(f, n), HID) for n in names]
    assert torch.equal(q, torch.cat([a for a, _ in by_hand])) and torch.equal(s, torch.cat([b for _, b in by_hand]))
    assert (cache.hits, cache.misses) == (0, 1)
    q2, s2 = loader.w8a8_linear(f, names, HID, cache=cache)
    assert (cache.hits, cache.misses) == (1, 1) and torch.equal(q, q2) and torch.equal(s, s2)
    # a different parameter is a different blob: Q8_0's own groups keep the file's bytes
    q32, s32 = loader.w8a8_linear(f, names, 32, cache=cache)
    assert cache.misses == 2 and s32.shape == (QC + 2 * KVC, HID // 32)
    assert torch.equal(q32[:QC], loader.tensor(f, names[0]).qs)
    smooth = torch.exp(torch.randn(HID, generator=torch.Generator().manual_seed(3)) * 0.1)
    qs_, _ = loader.w8a8_linear(f, names, HID, smooth=smooth, cache=cache)
    assert cache.misses == 3 and not torch.equal(qs_, q)
    # W4A8: layer 1's q, k (Q4_K) and v (Q6_K) become two segments
    names1 = [f"blk.1.{s}" for s in loader.LAYER_TENSORS["qkv"]]
    segs = loader.w4a8_linear(f, names1, "cpu", cache=cache)
    assert [(w.kind, w.n, first) for w, first in segs] == [("q4k", QC + KVC, 0), ("q6k", KVC, QC + KVC)]
    direct = w4a8.segments([loader.tensor(f, n) for n in names1], "cpu")
    for (a, fa), (b, fb) in zip(segs, direct):
        assert fa == fb and all((x is None and y is None) or torch.equal(x, y)
                                for x, y in zip((a.q, a.sc, a.mn, a.d, a.dm), (b.q, b.sc, b.mn, b.d, b.dm)))
    again = loader.w4a8_linear(f, names1, "cpu", cache=cache)
    assert cache.hits == 2 and torch.equal(again[1][0].q, segs[1][0].q)
    # a k-quant tensor on the W8A8 path goes through Q8_0 blocks of its dequantized values
    qk, sk = loader.w8a8_linear(f, [names1[2]], 32, cache=cache)
    assert torch.equal(qk, loader.tensor(f, names1[2]).as_q8().qs)
    # MXFP4 from the dequantized weights
    m = loader.mxfp4_linear(f, [f"blk.0.{s}" for s in loader.LAYER_TENSORS["down"]], cache=cache)
    want = mxfp4.pack(loader.tensor(f, "blk.0.ffn_down.weight").dequant(), "max")
    assert m.shape == (HID, FFN) and torch.equal(m.q, want.q) and torch.equal(m.s, want.s)
    # the whole layer, as LinearStack takes it
    layer = loader.layer_linear_set(f, 0, "cpu", cache=cache)
    assert layer["qkv"][0].shape == (QC + 2 * KVC, HID) and layer["gate_up"][0].shape == (2 * FFN, HID)
    assert layer["down"][0].shape == (HID, FFN) and layer["o"][1].shape == (HID,)
    # touching the file invalidates every key
    os.utime(path, ns=(1, 1))
    loader.w8a8_linear(G.GGUFFile(path), names, HID, cache=cache)
    assert cache.misses >= 7
