"""Reading and writing the safetensors container: an 8-byte little-endian header length, a JSON
directory ``name -> {dtype, shape, data_offsets}``, then the raw tensor bytes.

Role of the reference's GGUF reader (``gguf_open``, fastgguf.c:342-440): parse the directory
with bounds checks, reject unsupported types by name (:421-425), reject tensors that reach past
the end of the file (:432-435), and find tensors by exact name (``tensor_find``, :456-460).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; ``tensor(name)`` gives a CPU tensor viewing the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {})
        self._data0 = 8 + hlen
        data_size = size - self._data0
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: tensor '{name}' has a malformed directory entry") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}': unsupported type {dt}")
            n = 1
            for s in shape:
                n *= s
            if b < 0 or e < b or e > data_size:
                raise SafetensorsError(f"{path}: tensor '{name}' extends past the end of the file")
            if e - b != n * _DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' of shape {list(shape)} {dt} needs {n * _DTYPES[dt][1]} bytes, "
                    f"its directory entry gives {e - b}")
            self.entries[name] = TensorEntry(name, _DTYPES[dt][0], shape, b, e)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        n = 1
        for s in e.shape:
            n *= s
        if n == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._map)[self._data0 + e.begin:self._data0 + e.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the map is read-only; the tensor is only read
            t = torch.frombuffer(buf, dtype=e.dtype)
        return t.reshape(e.shape)

    def close(self) -> None:
        # tensors handed out keep the map alive through their buffer; only drop our handles
        self._map = None
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write CPU tensors in name order, data aligned so the header is a multiple of 8 bytes."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
