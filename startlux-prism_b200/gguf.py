"""GGUF (versions 2 and 3) container reader: metadata, tensor directory and raw tensor bytes.  The counterpart of the
reference's startlux_prism/gguf.py:30-95 (GGUFFile, BLOCK): the same public surface - `meta`, `tensors[name]` with
`dims` in ggml order (dims[0] is the contiguous input dimension), `type`, absolute `offset`, `nbytes`, and
`read(name) -> uint8 array` - so code written against the reference's reader runs on this one.

The header is parsed from one memory map with struct.unpack_from (a cursor over bytes, no per-field file reads);
tensor data is read with one positioned read per tensor into a fresh array, never kept mapped.
"""
from __future__ import annotations

import dataclasses
import mmap
import struct

import numpy as np

GGML_F32, GGML_F16, GGML_Q8_0, GGML_BF16 = 0, 1, 8, 30
GGML_Q4_K, GGML_Q5_K, GGML_Q6_K = 12, 13, 14
# ggml type -> (elements per block, bytes per block)
BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q8_0: (32, 34),
         GGML_Q4_K: (256, 144), GGML_Q5_K: (256, 176), GGML_Q6_K: (256, 210)}
TYPE_NAMES = {GGML_F32: "F32", GGML_F16: "F16", GGML_BF16: "BF16", GGML_Q8_0: "Q8_0", GGML_Q4_K: "Q4_K",
              GGML_Q5_K: "Q5_K", GGML_Q6_K: "Q6_K"}

# GGUF metadata value types: fixed-size scalars by struct code; 8 = string, 9 = array
_FIXED = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}
_STRING, _ARRAY = 8, 9


@dataclasses.dataclass(frozen=True)
class TensorInfo:
    name: str
    dims: tuple
    type: int
    offset: int
    nbytes: int

    @property
    def shape(self):
        """[outputs..., inputs]: the row-major shape (ggml's dims reversed)."""
        return tuple(int(d) for d in reversed(self.dims))


class _Cursor:
    """Sequential little-endian reads over a bytes-like object."""

    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, code):
        (v,) = struct.unpack_from("<" + code, self.buf, self.pos)
        self.pos += struct.calcsize(code)
        return v

    def string(self):
        n = self.take("Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, kind):
        if kind in _FIXED:
            return self.take(_FIXED[kind])
        if kind == _STRING:
            return self.string()
        if kind == _ARRAY:
            inner, n = self.take("I"), self.take("Q")
            if inner in _FIXED:
                dt = np.dtype("<" + _FIXED[inner]) if inner != 7 else np.dtype(np.bool_)
                out = np.frombuffer(self.buf, dtype=dt, count=n, offset=self.pos)
                self.pos += dt.itemsize * n
                return out.tolist()
            return [self.value(inner) for _ in range(n)]
        raise ValueError(f"GGUF metadata value type {kind} is unknown")


class GGUFFile:
    """meta: dict key -> value; tensors: dict name -> TensorInfo (file order kept); version: 2 or 3."""

    def __init__(self, path):
        self.path = str(path)
        with open(self.path, "rb") as f:
            size = f.seek(0, 2)
            if size < 24:
                raise ValueError(f"{path}: not a GGUF file")
            with mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as m:
                if m[:4] != b"GGUF":
                    raise ValueError(f"{path}: not a GGUF file")
                c = _Cursor(m)
                c.pos = 4
                self.version = c.take("I")
                if self.version not in (2, 3):
                    raise ValueError(f"{path}: GGUF version {self.version} not supported")
                n_tensors, n_meta = c.take("Q"), c.take("Q")
                self.meta = {}
                for _ in range(n_meta):
                    key = c.string()
                    self.meta[key] = c.value(c.take("I"))
                directory = []
                for _ in range(n_tensors):
                    name = c.string()
                    dims = tuple(c.take("Q") for _ in range(c.take("I")))
                    directory.append((name, dims, c.take("I"), c.take("Q")))
                header_end = c.pos
        align = int(self.meta.get("general.alignment", 32))
        data0 = (header_end + align - 1) // align * align
        self.tensors = {}
        for name, dims, typ, rel in directory:
            if typ not in BLOCK:
                raise ValueError(f"{name}: ggml type {typ} not supported")
            per, nb = BLOCK[typ]
            count = 1
            for d in dims:
                count *= int(d)
            if dims and int(dims[0]) % per:
                raise ValueError(f"{name}: {dims[0]} inputs are not whole {TYPE_NAMES[typ]} blocks")
            info = TensorInfo(name, dims, typ, data0 + rel, count // per * nb)
            if info.offset + info.nbytes > size:
                raise ValueError(f"{name}: truncated file")
            self.tensors[name] = info

    def read(self, name):
        """The tensor's bytes as a fresh uint8 array."""
        t = self.tensors[name]
        buf = np.fromfile(self.path, dtype=np.uint8, count=t.nbytes, offset=t.offset)
        if buf.size != t.nbytes:
            raise ValueError(f"{name}: truncated file")
        return buf
