"""Reading and writing the safetensors container: eight bytes of header
length, a JSON header (name -> dtype, shape, data_offsets), then the raw
little-endian data.  Own code; no model library is involved.

Reference counterpart: the GGUF header scan that builds name -> (offset,
type, dims) in ``src/backend/bindless/metadata.rs:82-108``.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a readable safetensors container."""


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """One file, memory-mapped; tensors are read on demand."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short for a safetensors header")
        self._fh = open(self.path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from e
        self._base = 8 + hlen
        self.entries = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (a, b) = meta["dtype"], tuple(meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: malformed entry for '{name}'") from None
            if dtype not in DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {dtype}")
            nbytes = _numel(shape) * torch.empty(0, dtype=DTYPES[dtype]).element_size()
            if a < 0 or b < a or b - a != nbytes or self._base + b > size:
                raise SafetensorsError(f"{self.path}: tensor '{name}' data range [{a}, {b}) does not "
                                       f"match its shape {list(shape)} or lies outside the file")
            self.entries[name] = (dtype, shape, a, b)
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return list(self.entries)

    def info(self, name):
        dtype, shape, _, _ = self.entries[name]
        return DTYPES[dtype], shape

    def read(self, name) -> torch.Tensor:
        dtype, shape, a, b = self.entries[name]
        if b == a:
            return torch.empty(shape, dtype=DTYPES[dtype])
        buf = bytearray(self._mm[self._base + a: self._base + b])
        return torch.frombuffer(buf, dtype=DTYPES[dtype]).reshape(shape)

    def close(self):
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._fh.close()


def write_safetensors(path, tensors, metadata=None) -> None:
    """Write ``tensors`` (an iterable of ``(name, shape, dtype, make)`` where
    ``make()`` returns the CPU tensor) to ``path``.  The header is written
    first from the declared shapes; tensors are produced one at a time."""
    items = list(tensors)
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, shape, dtype, _ in items:
        n = _numel(shape) * torch.empty(0, dtype=dtype).element_size()
        header[name] = {"dtype": NAMES[dtype], "shape": [int(s) for s in shape], "data_offsets": [off, off + n]}
        off += n
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(raw)))
        fh.write(raw)
        for name, shape, dtype, make in items:
            t = make()
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise SafetensorsError(f"tensor '{name}': made {list(t.shape)} {t.dtype}, "
                                       f"declared {list(shape)} {dtype}")
            t = t.contiguous().cpu()
            if t.numel():
                fh.write(t.view(torch.uint8).numpy().data)      # (the array's own memory: no copy)
