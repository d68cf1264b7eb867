"""GGUF tensor files -> weights resident in HBM.

A reader for the GGUF container (versions 2 and 3: magic, header, metadata key/values, tensor table, aligned data
section) that memory-maps the file and hands each quantized tensor's blocks — already in the layout the kernels'
repacker takes: n rows of k / block_size blocks, the reference's `#[repr(C)]` block structs (src/quant.rs:122-157,
254-293) being the GGUF block layouts — to `GpuKernels.upload`.  F32 / F16 tensors come back as numpy arrays.
`write_gguf` produces a minimal file (used by the tests and for exporting synthetic checkpoints).

ggml tensor types served: Q4_0 (2), Q5_0 (6), Q8_0 (8), Q4_K (12), Q5_K (13), Q6_K (14), Q8_K (15), F32 (0), F16 (1).
Anything else is listed by `tensors()` and refused by `load()` with the type id in the message.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np

from .quant import QuantType

GGUF_MAGIC = 0x46554747  # "GGUF", little-endian
DEFAULT_ALIGNMENT = 32

GGML_F32, GGML_F16 = 0, 1
# ggml type id -> QuantType constructor
_QUANT = {2: QuantType.q4_0, 6: QuantType.q5_0, 8: QuantType.q8_0, 12: QuantType.q4k, 13: QuantType.q5k,
          14: QuantType.q6k, 15: QuantType.q8k}
_GGML_OF = {8: 2, 9: 6, 2: 8, 1: 12, 7: 13, 6: 14, 10: 15}  # QuantType.id -> ggml type id

# metadata value types
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class GgufError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple       # ggml order: shape[0] is the row length k (innermost), shape[1] the number of rows n
    ggml_type: int
    offset: int        # from the start of the data section
    nbytes: int

    @property
    def k(self) -> int:
        return int(self.shape[0])

    @property
    def n(self) -> int:
        r = 1
        for d in self.shape[1:]:
            r *= int(d)
        return r

    @property
    def quant_type(self):
        f = _QUANT.get(self.ggml_type)
        return f() if f else None


def _tensor_bytes(ggml_type: int, shape) -> int:
    count = 1
    for d in shape:
        count *= int(d)
    if ggml_type == GGML_F32:
        return 4 * count
    if ggml_type == GGML_F16:
        return 2 * count
    f = _QUANT.get(ggml_type)
    if f is None:
        return -1
    qt = f()
    if int(shape[0]) % qt.block_size():
        raise GgufError(f"row length {shape[0]} is not a multiple of the block size {qt.block_size()}")
    return count // qt.block_size() * qt.block_bytes()


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("truncated file")
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if n > (1 << 24) or self.pos + n > len(self.buf):
            raise GgufError("bad string length")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype in _SCALARS:
            return self.take(_SCALARS[vtype])
        if vtype == _T_STRING:
            return self.string()
        if vtype == _T_ARRAY:
            et, n = self.take("<I"), self.take("<Q")
            if n > (1 << 28):
                raise GgufError("bad array length")
            return [self.value(et) for _ in range(n)]
        raise GgufError(f"unknown metadata value type {vtype}")


class GgufFile:
    """Memory-mapped GGUF file: `metadata` (dict), `tensors()` (name -> TensorInfo), `raw(name)`, `load(K, name)`."""

    def __init__(self, path: str):
        self._f = open(path, "rb")
        try:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError as e:
            self._f.close()
            raise GgufError(f"cannot map {path}: {e}") from e
        c = _Cursor(self._mm)
        if c.take("<I") != GGUF_MAGIC:
            self.close()
            raise GgufError("not a GGUF file (bad magic)")
        self.version = c.take("<I")
        if self.version not in (2, 3):
            self.close()
            raise GgufError(f"unsupported GGUF version {self.version}")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        if n_tensors > (1 << 20) or n_kv > (1 << 20):
            self.close()
            raise GgufError("implausible tensor / metadata count")
        self.metadata = {}
        for _ in range(n_kv):
            key = c.string()
            self.metadata[key] = c.value(c.take("<I"))
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        if self.alignment <= 0 or self.alignment & (self.alignment - 1):
            self.close()
            raise GgufError(f"alignment {self.alignment} is not a power of two")
        self._tensors = {}
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            if nd < 1 or nd > 4:
                self.close()
                raise GgufError(f"tensor {name}: {nd} dimensions")
            shape = tuple(c.take("<Q") for _ in range(nd))
            gt, off = c.take("<I"), c.take("<Q")
            self._tensors[name] = TensorInfo(name, shape, gt, off, _tensor_bytes(gt, shape))
        self.data_start = (c.pos + self.alignment - 1) // self.alignment * self.alignment
        for t in self._tensors.values():
            if t.offset % self.alignment:
                self.close()
                raise GgufError(f"tensor {t.name}: offset {t.offset} is not aligned to {self.alignment}")
            if t.nbytes >= 0 and self.data_start + t.offset + t.nbytes > len(self._mm):
                self.close()
                raise GgufError(f"tensor {t.name}: data runs past the end of the file")

    def close(self) -> None:
        if getattr(self, "_mm", None) is not None:
            try:
                self._mm.close()
            except BufferError:  # a caller still holds a view from raw(): the mapping goes when the view does
                pass
            self._mm = None
        if getattr(self, "_f", None) is not None:
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def tensors(self) -> dict:
        return dict(self._tensors)

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a read-only uint8 view of the mapping (no copy)."""
        t = self._tensors[name]
        if t.nbytes < 0:
            raise GgufError(f"tensor {name}: ggml type {t.ggml_type} is not served")
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=self.data_start + t.offset)

    def load(self, K, name: str):
        """Quantized tensor -> `Weight` in HBM (repacked once by `K.upload`); F32 / F16 -> numpy array [n, k] (a copy)."""
        t = self._tensors[name]
        if t.ggml_type == GGML_F32:
            return self.raw(name).view(np.float32).reshape(t.n, t.k).copy()
        if t.ggml_type == GGML_F16:
            return self.raw(name).view(np.float16).reshape(t.n, t.k).copy()
        qt = t.quant_type
        if qt is None:
            raise GgufError(f"tensor {name}: ggml type {t.ggml_type} is not served")
        return K.upload(qt, t.n, t.k, np.ascontiguousarray(self.raw(name)))

    def load_all(self, K, names=None) -> dict:
        """Every served tensor (or the named ones) -> {name: Weight | ndarray}."""
        out = {}
        for name, t in self._tensors.items():
            if names is not None and name not in names:
                continue
            if t.nbytes >= 0:
                out[name] = self.load(K, name)
        return out


def write_gguf(path: str, tensors: dict, metadata: dict | None = None, alignment: int = DEFAULT_ALIGNMENT) -> None:
    """tensors: name -> (QuantType, n, k, blocks uint8) or a float32 / float16 array [n, k]; metadata: str -> int |
    float | str | bool (written as u32 / i64, f32, string, bool)."""
    def s(x: str) -> bytes:
        b = x.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    md = dict(metadata or {})
    md["general.alignment"] = alignment
    kv = b""
    for key, v in md.items():
        kv += s(key)
        if isinstance(v, bool):
            kv += struct.pack("<I?", 7, v)
        elif isinstance(v, int):
            kv += struct.pack("<II", 4, v) if 0 <= v < (1 << 32) else struct.pack("<Iq", 11, v)
        elif isinstance(v, float):
            kv += struct.pack("<If", 6, v)
        else:
            kv += struct.pack("<I", _T_STRING) + s(str(v))
    infos, blobs, off = b"", [], 0
    for name, t in tensors.items():
        if isinstance(t, tuple):
            qt, n, k, blocks = t
            data = np.ascontiguousarray(blocks, dtype=np.uint8).tobytes()
            if len(data) != n * (k // qt.block_size()) * qt.block_bytes():
                raise GgufError(f"tensor {name}: {len(data)} bytes for [{n}, {k}] {qt.name}")
            gt = _GGML_OF[qt.id]
        else:
            a = np.ascontiguousarray(t)
            if a.dtype not in (np.float32, np.float16) or a.ndim != 2:
                raise GgufError(f"tensor {name}: expected a 2-D float32 / float16 array")
            n, k = a.shape
            data, gt = a.tobytes(), (GGML_F32 if a.dtype == np.float32 else GGML_F16)
        infos += s(name) + struct.pack("<IQQIQ", 2, k, n, gt, off)
        blobs.append((off, data))
        off = (off + len(data) + alignment - 1) // alignment * alignment
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(md)) + kv + infos
    start = (len(head) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * (start - len(head)))
        for o, data in blobs:
            f.seek(start + o)
            f.write(data)
        f.truncate(start + off if blobs else start)
