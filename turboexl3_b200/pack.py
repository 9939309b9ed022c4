"""Reading an EXL3 pack from safetensors files (host side, numpy only).

The reference's plugin is handed the pack's tensors by its host, which reads them from safetensors shards: a trunk linear
is `<base>.weight` (the trellis, u16/i16 [in/16, out/16, n]) beside `<base>.scales` (suh f16 [in]) and `<base>.biases`
(svh f16 [out]); a routed bank is `<base>.trellis` (u16 [E, in/16, out/16, n]), `<base>.suh` (f16 [E, in]) and `<base>.svh`
(f16 [E, out]) (table/table.zig:126-172). This module is that host-side step for callers of this library: it maps the
files, finds the three tensors of a base name and returns them as arrays the table's `load_tensor` / `load_bank` take
(no copy: the arrays are views of the mapped file; the table uploads them once).

safetensors layout: 8 bytes little-endian header length N, N bytes of JSON {name: {"dtype", "shape", "data_offsets":
[begin, end]}, "__metadata__": {...}}, then the tensors' bytes; offsets count from the end of the header.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np

_DTYPES = {"F16": np.float16, "F32": np.float32, "U16": np.uint16, "I16": np.int16, "I32": np.int32, "U32": np.uint32,
           "U8": np.uint8, "I8": np.int8, "F64": np.float64, "I64": np.int64, "U64": np.uint64, "BOOL": np.bool_}
_NAMES = {np.dtype(v).str: k for k, v in _DTYPES.items()}


class PackError(ValueError):
    pass


class Shard:
    """One mapped safetensors file. Tensors come back as read-only views of the mapping. bf16 tensors (no numpy dtype)
    come back as uint16 bit patterns with `dtype_of(name) == "BF16"`."""

    def __init__(self, path: str):
        self.path = path
        self._file = open(path, "rb")
        size = os.fstat(self._file.fileno()).st_size
        if size < 8:
            raise PackError(f"{path}: not a safetensors file")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._map[:8])
        if n > size - 8:
            raise PackError(f"{path}: header length {n} exceeds the file")
        header = json.loads(bytes(self._map[8:8 + n]).decode("utf-8"))
        self.metadata = header.pop("__metadata__", {})
        self._entries = header
        self._base = 8 + n
        for name, e in header.items():
            b, end = e["data_offsets"]
            if not (0 <= b <= end <= size - self._base):
                raise PackError(f"{path}: tensor {name} lies outside the file")

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def dtype_of(self, name: str) -> str:
        return self._entries[name]["dtype"]

    def tensor(self, name: str) -> np.ndarray:
        e = self._entries[name]
        dt = np.uint16 if e["dtype"] == "BF16" else _DTYPES.get(e["dtype"])
        if dt is None:
            raise PackError(f"{self.path}: tensor {name} has dtype {e['dtype']}")
        b, end = e["data_offsets"]
        count = int(np.prod(e["shape"], dtype=np.int64)) if e["shape"] else 1
        if (end - b) != count * np.dtype(dt).itemsize:
            raise PackError(f"{self.path}: tensor {name} has {end - b} bytes for shape {e['shape']}")
        return np.frombuffer(self._map, dtype=dt, count=count, offset=self._base + b).reshape(e["shape"])

    def close(self) -> None:
        self._map.close()
        self._file.close()


class Pack:
    """The shards of a pack directory (every *.safetensors file), one name space."""

    def __init__(self, paths: Iterable[str]):
        self.shards = [Shard(p) for p in paths]
        self._where: Dict[str, Shard] = {}
        for sh in self.shards:
            for name in sh.names():
                self._where[name] = sh

    @classmethod
    def open_dir(cls, directory: str) -> "Pack":
        return cls(sorted(os.path.join(directory, f) for f in os.listdir(directory) if f.endswith(".safetensors")))

    def has(self, name: str) -> bool:
        return name in self._where

    def tensor(self, name: str) -> np.ndarray:
        if name not in self._where:
            raise PackError(f"MissingWeight: {name}")  # the refusal the reference's loader gives (table/table.zig:133)
        return self._where[name].tensor(name)

    def trunk(self, base: str) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
        """(trellis, suh, svh) of a trunk linear stored under the affine names (table/table.zig:126-148)."""
        t = self.tensor(base + ".weight")
        return t.view(np.uint16) if t.dtype == np.int16 else t, self.tensor(base + ".scales"), self.tensor(base + ".biases")

    def bank(self, base: str) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
        """(trellis, suh, svh) of a routed bank (table/table.zig:157-172)."""
        return self.tensor(base + ".trellis"), self.tensor(base + ".suh"), self.tensor(base + ".svh")

    def close(self) -> None:
        for sh in self.shards:
            sh.close()


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], metadata: Dict[str, str] | None = None) -> None:
    """Writes a safetensors file (for tests and for packing synthetic operands)."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        key = _NAMES.get(a.dtype.str)
        if key is None:
            raise PackError(f"dtype {a.dtype} has no safetensors name")
        header[name] = {"dtype": key, "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        blobs.append(a.tobytes())
        off += a.nbytes
    if metadata:
        header["__metadata__"] = metadata
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for b in blobs:
            f.write(b)
