"""From a GGUF file's tensors to the layouts the kernels read, with an on-disk cache of the converted blobs.

The reference converts at every start, in Python, inside its engine: tensor bytes -> Q8 / KQuant containers
(gguf_weights.py:221-244, the `get` of :270-279), Q8_0 -> int8 rows with one scale per group or per row and optional
SmoothQuant factors (kernels/w8a8.py:274-286, engine/model.py:72-82), k-quants -> the W4A8 repack (kernels/w4a8.py:70-94),
any matrix -> MXFP4 codes with a side file beside the model (engine/mxfp4.py:46-82).  This module does the same
conversions per projection and keeps each result in a cache directory, keyed by the file's identity (path, size,
modification time), the tensor names, the layout's name and parameters and LAYOUT_VERSION: a second start reads the
blobs back instead of converting.

    f = gguf.GGUFFile(path)
    tensor(f, "blk.0.ffn_down.weight")                   -> Q8 | KQuant | fp32 tensor
    w8a8_linear(f, names, gk, smooth=None, cache=None)   -> (int8 [N, K], fp32 [N, K / gk])   rows of `names` stacked
    w4a8_linear(f, names, device, cache=None)            -> [(w4a8.W4, first output column)]  (w4a8.gemm_segs)
    mxfp4_linear(f, names, mode="max", cache=None)       -> mxfp4.MX4 (CPU; mxfp4.prepare() on the device)
    layer_linear_set(f, i, device, gk=None, cache=None)  -> the dict LinearStack takes for layer i (W8A8)
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import torch

from . import gguf as G
from . import gguf_weights as GW

LAYOUT_VERSION = 1
K_QUANTS = (G.GGML_Q4_K, G.GGML_Q5_K, G.GGML_Q6_K)


def tensor(f: G.GGUFFile, name):
    """One tensor of the file in its container: Q8_0 -> gguf_weights.Q8 (qs int8 [n, k], d fp16 [n, k / 32]), k-quants ->
    gguf_weights.KQuant (raw super-blocks [n, k / 256, block bytes]), F32 / F16 / BF16 -> a torch tensor in row-major
    shape (fp32 for F32, else the stored type)."""
    t = f.tensors[name]
    k = int(t.dims[0])
    n = 1
    for d in t.dims[1:]:
        n *= int(d)
    raw = torch.from_numpy(f.read(name))
    if t.type == G.GGML_Q8_0:
        return GW.Q8.from_blocks(raw, n, k)
    if t.type in K_QUANTS:
        per, nb = G.BLOCK[t.type]
        return GW.KQuant(raw.reshape(n, k // per, nb), t.type, k)
    if t.type == G.GGML_F32:
        return raw.view(torch.float32).reshape(t.shape).clone()
    if t.type == G.GGML_F16:
        return raw.view(torch.float16).reshape(t.shape).clone()
    if t.type == G.GGML_BF16:
        return raw.view(torch.bfloat16).reshape(t.shape).clone()
    raise ValueError(f"{name}: ggml type {t.type} has no container here")


class LayoutCache:
    """A directory of converted blobs.  A key names everything the blob depends on; the blob is a dict of tensors
    written with torch.save to a temporary name and renamed into place (ranks that start together may both convert;
    whichever renames last wins with identical bytes)."""

    def __init__(self, directory):
        self.dir = str(directory)
        os.makedirs(self.dir, exist_ok=True)
        self.hits = self.misses = 0

    @staticmethod
    def key(f: G.GGUFFile, names, layout, **params):
        st = os.stat(f.path)
        ident = {"file": os.path.abspath(f.path), "size": st.st_size, "mtime_ns": st.st_mtime_ns, "tensors": list(names),
                 "layout": layout, "version": LAYOUT_VERSION,
                 "params": {k: (v if isinstance(v, (int, float, str, type(None))) else _digest(v)) for k, v in sorted(params.items())}}
        return hashlib.sha256(json.dumps(ident, sort_keys=True).encode()).hexdigest()[:32]

    def path(self, key):
        return os.path.join(self.dir, key + ".pt")

    def get(self, key):
        p = self.path(key)
        if not os.path.exists(p):
            self.misses += 1
            return None
        self.hits += 1
        return torch.load(p, map_location="cpu", weights_only=True)

    def put(self, key, blob):
        tmp = self.path(key) + f".tmp{os.getpid()}"
        torch.save(blob, tmp)
        os.replace(tmp, self.path(key))


def _digest(t):
    """A short content hash of a tensor parameter (SmoothQuant factors change the converted weights)."""
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return hashlib.sha256(a.tobytes()).hexdigest()[:16]


def _cached(cache, f, names, layout, build, **params):
    if cache is None:
        return build()
    key = cache.key(f, names, layout, **params)
    blob = cache.get(key)
    if blob is None:
        blob = build()
        cache.put(key, blob)
    return blob


def _as_q8(x, name):
    if isinstance(x, GW.Q8):
        return x
    if isinstance(x, GW.KQuant):
        return x.as_q8()                      # a k-quant tensor on the W8A8 path: its values as Q8_0 blocks
    raise ValueError(f"{name}: a float tensor is not a quantized projection")


def w8a8_linear(f, names, gk, smooth=None, cache=None):
    """The matrices `names` (stacked top to bottom: a fused projection) as W8A8 weights: int8 [N, K] and fp32 scales
    [N, K / gk]; gk == K gives one scale per output row (the engine's mode), gk == 32 keeps Q8_0's own values and block
    scales.  smooth fp32 [K]: SmoothQuant factors multiplied into the weights before they are quantized again."""
    from . import w8a8

    def build():
        qs, ss = [], []
        for name in names:
            q, s = w8a8.weight_from_q8(_as_q8(tensor(f, name), name), gk, smooth)
            qs.append(q)
            ss.append(s)
        return {"q": torch.cat(qs, 0).contiguous(), "s": torch.cat(ss, 0).contiguous()}
    blob = _cached(cache, f, names, "w8a8", build, gk=gk, smooth=smooth)
    return blob["q"], blob["s"]


def w4a8_linear(f, names, device, cache=None):
    """The k-quant matrices `names` as the segments of one fused W4A8 projection (neighbours of one kind fused), on
    `device`."""
    from . import w4a8

    def build():
        segs = w4a8.segments([tensor(f, name) for name in names], "cpu")
        blob = {"n": torch.tensor(len(segs))}
        for i, (w, first) in enumerate(segs):
            blob[f"{i}.meta"] = torch.tensor([0 if w.kind == "q4k" else 1, w.n, w.k, first])
            for field in ("q", "sc", "mn", "d", "dm"):
                t = getattr(w, field)
                if t is not None:
                    blob[f"{i}.{field}"] = t
        return blob
    blob = _cached(cache, f, names, "w4a8", build)
    segs = []
    for i in range(int(blob["n"])):
        kind, n, k, first = (int(v) for v in blob[f"{i}.meta"])
        get = lambda field: blob[f"{i}.{field}"].to(device) if f"{i}.{field}" in blob else None   # noqa: E731
        segs.append((w4a8.W4("q4k" if kind == 0 else "q6k", get("q"), get("sc"), get("mn"), get("d"), get("dm"), n, k), first))
    return segs


def mxfp4_linear(f, names, mode="max", cache=None):
    """The matrices `names` (stacked) requantized to MXFP4 from their dequantized values (mxfp4.pack): codes uint8
    [N, K / 2], UE8M0 scales uint8 [N, K / 32].  On the CPU; move it to the device and mxfp4.prepare() it there."""
    from . import mxfp4

    def build():
        parts = []
        for name in names:
            x = tensor(f, name)
            parts.append(x.dequant(torch.float32) if isinstance(x, (GW.Q8, GW.KQuant)) else x.float())
        w = mxfp4.pack(torch.cat(parts, 0), mode)
        return {"q": w.q, "s": w.s, "shape": torch.tensor([w.n, w.k])}
    blob = _cached(cache, f, names, "mxfp4", build, mode=mode)
    n, k = (int(v) for v in blob["shape"])
    return mxfp4.MX4(blob["q"], blob["s"], n, k)


# tensor names of a decoder layer's linear set in a llama.cpp-style GGUF file (gguf_weights.py:281-293)
LAYER_TENSORS = {"qkv": ("attn_q.weight", "attn_k.weight", "attn_v.weight"), "o": ("attn_output.weight",),
                 "gate_up": ("ffn_gate.weight", "ffn_up.weight"), "down": ("ffn_down.weight",)}


def layer_linear_set(f, layer, device, gk=None, cache=None):
    """Layer `layer`'s q|k|v, o, gate|up and down projections as the W8A8 weights linear_stack.LinearStack takes:
    dict name -> (int8 [N, K], fp32 [N]) on `device` (gk None: one scale per output row)."""
    out = {}
    for key, suffixes in LAYER_TENSORS.items():
        names = [f"blk.{layer}.{s}" for s in suffixes]
        k = int(f.tensors[names[0]].dims[0])
        q, s = w8a8_linear(f, names, k if gk is None else gk, cache=cache)
        out[key] = (q.to(device), (s.view(-1) if gk is None else s).to(device))
    return out
