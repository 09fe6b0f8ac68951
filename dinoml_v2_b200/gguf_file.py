"""Minimal GGUF (v2/v3) container reader and writer: just enough to pull the raw encoded bytes of a
tensor out of a `.gguf` file (memory-mapped) and to write small files for tests and tools.

It stands in for the three libgguf calls the reference makes when it binds a GGUF constant -
`open_gguf`, `get_tensor`, `read_tensor_bytes` (src/dinoml/constant_sources.py:303-333).  The layout
follows the public GGUF specification: header (magic "GGUF", version, tensor count, key/value count),
key/value pairs, tensor infos (name, dims, ggml type, offset), padding to `general.alignment`
(default 32), tensor data.  GGUF stores dimensions innermost-first, so a `[N, K]` weight has GGUF
shape `[K, N]` (the reference reverses it the same way, src/dinoml/constant_sources.py:336-339).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np

GGUF_MAGIC = b"GGUF"
DEFAULT_ALIGNMENT = 32

# ggml type id -> (name, block size, block bytes)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 8: ("Q8_0", 32, 34), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110),
    12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 30: ("BF16", 1, 2), 39: ("MXFP4", 32, 17),
    40: ("NVFP4", 64, 36),
}
_TYPE_ID = {name: tid for tid, (name, _, _) in GGML_TYPES.items()}

# GGUF metadata value types
_U8, _I8, _U16, _I16, _U32, _I32, _F32, _BOOL, _STR, _ARR, _U64, _I64, _F64 = range(13)
_SCALAR = {_U8: "<B", _I8: "<b", _U16: "<H", _I16: "<h", _U32: "<I", _I32: "<i", _F32: "<f", _BOOL: "<?",
           _U64: "<Q", _I64: "<q", _F64: "<d"}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple[int, ...]       # GGUF order (innermost first)
    qtype_value: int
    qtype: str
    data_offset: int             # absolute file offset of the first byte
    nbytes: int


class GGUFFile:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self._fh = open(self.path, "rb")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        self.metadata: dict[str, Any] = {}
        self.tensors: dict[str, TensorInfo] = {}
        self._parse()

    # -- parsing helpers
    def _unpack(self, fmt: str):
        size = struct.calcsize(fmt)
        value = struct.unpack_from(fmt, self._mm, self._pos)[0]
        self._pos += size
        return value

    def _string(self) -> str:
        n = self._unpack("<Q")
        s = bytes(self._mm[self._pos:self._pos + n]).decode("utf-8")
        self._pos += n
        return s

    def _value(self, vtype: int):
        if vtype in _SCALAR:
            return self._unpack(_SCALAR[vtype])
        if vtype == _STR:
            return self._string()
        if vtype == _ARR:
            etype = self._unpack("<I")
            count = self._unpack("<Q")
            return [self._value(etype) for _ in range(count)]
        raise ValueError(f"{self.path}: unknown GGUF metadata value type {vtype}")

    def _parse(self) -> None:
        self._pos = 0
        if bytes(self._mm[0:4]) != GGUF_MAGIC:
            raise ValueError(f"{self.path} is not a GGUF file")
        self._pos = 4
        self.version = self._unpack("<I")
        if self.version not in (2, 3):
            raise ValueError(f"{self.path}: unsupported GGUF version {self.version}")
        n_tensors = self._unpack("<Q")
        n_kv = self._unpack("<Q")
        for _ in range(n_kv):
            key = self._string()
            self.metadata[key] = self._value(self._unpack("<I"))
        infos = []
        for _ in range(n_tensors):
            name = self._string()
            ndim = self._unpack("<I")
            shape = tuple(self._unpack("<Q") for _ in range(ndim))
            tid = self._unpack("<I")
            rel = self._unpack("<Q")
            infos.append((name, shape, tid, rel))
        align = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        data_start = (self._pos + align - 1) // align * align
        for name, shape, tid, rel in infos:
            tname, bs, bb = GGML_TYPES.get(tid, (f"TYPE_{tid}", 0, 0))
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            nbytes = numel // bs * bb if bs else 0
            self.tensors[name] = TensorInfo(name, shape, tid, tname, data_start + rel, nbytes)

    # -- the three calls the constant binder needs
    def get_tensor(self, name: str) -> TensorInfo | None:
        return self.tensors.get(name)

    def read_tensor_bytes(self, info: TensorInfo) -> memoryview:
        if info.nbytes == 0:
            raise ValueError(f"tensor {info.name!r} has unsupported ggml type {info.qtype}")
        return memoryview(self._mm)[info.data_offset:info.data_offset + info.nbytes]

    def close(self) -> None:
        self._mm.close()
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def open_gguf(path: str | Path) -> GGUFFile:
    return GGUFFile(path)


def write_gguf(path: str | Path, tensors: dict[str, tuple[str, tuple[int, ...], np.ndarray]],
               metadata: dict[str, Any] | None = None, alignment: int = DEFAULT_ALIGNMENT) -> None:
    """tensors: name -> (qtype name, LOGICAL shape e.g. (N, K), raw uint8 bytes).  Writes GGUF v3."""
    metadata = dict(metadata or {})
    metadata.setdefault("general.architecture", "b200-gguf-test")
    metadata["general.alignment"] = int(alignment)

    def s(text: str) -> bytes:
        raw = text.encode("utf-8")
        return struct.pack("<Q", len(raw)) + raw

    out = bytearray(GGUF_MAGIC + struct.pack("<IQQ", 3, len(tensors), len(metadata)))
    for key, value in metadata.items():
        out += s(key)
        if isinstance(value, str):
            out += struct.pack("<I", _STR) + s(value)
        elif isinstance(value, bool):
            out += struct.pack("<I?", _BOOL, value)
        elif isinstance(value, int):
            out += struct.pack("<II", _U32, value)
        elif isinstance(value, float):
            out += struct.pack("<If", _F32, value)
        else:
            raise TypeError(f"unsupported metadata value for {key!r}")
    rel = 0
    blobs = []
    for name, (qtype, shape, data) in tensors.items():
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        gguf_shape = tuple(reversed(tuple(int(d) for d in shape)))
        out += s(name) + struct.pack("<I", len(gguf_shape))
        for d in gguf_shape:
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", _TYPE_ID[qtype], rel)
        blobs.append((rel, data))
        rel = (rel + data.nbytes + alignment - 1) // alignment * alignment
    out += b"\0" * ((-len(out)) % alignment)
    base = len(out)
    for off, data in blobs:
        out += b"\0" * (base + off - len(out))
        out += data.tobytes()
    Path(path).write_bytes(bytes(out))
