"""Reading and writing safetensors files without a third-party reader.

Layout of a file: an 8-byte little-endian length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the raw little-endian tensor data the offsets point into.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path

import torch

_DTYPES = {
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int  # offsets into the file
    end: int


class SafetensorsFile:
    """One open file; tensors are views of its memory map until copied."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._fh = open(self.path, "rb")
        head = self._fh.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if 8 + hlen > size:
            raise ValueError(f"{self.path}: header length {hlen} exceeds file size {size}")
        header = json.loads(self._fh.read(hlen))
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, TensorEntry] = {}
        base = 8 + hlen
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {info['dtype']}")
            lo, hi = info["data_offsets"]
            entry = TensorEntry(name, _DTYPES[info["dtype"]], tuple(info["shape"]), base + lo, base + hi)
            numel = 1
            for s in entry.shape:
                numel *= s
            if hi - lo != numel * entry.dtype.itemsize or base + hi > size:
                raise ValueError(f"{self.path}: tensor {name!r} has inconsistent offsets")
            self.entries[name] = entry
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes in the file."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the map is read-only; callers copy, never write
            flat = torch.frombuffer(memoryview(self._map)[e.begin : e.end], dtype=e.dtype)
        return flat.view(e.shape)

    def close(self) -> None:
        # tensors handed out may still view the map; it is unmapped when they are gone
        self._fh.close()


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    ordered = sorted(tensors)
    for name in ordered:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise ValueError(f"cannot store dtype {t.dtype} of {name!r}")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(len(blob) + 8) % 8)  # data starts on an 8-byte boundary
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in ordered:
            t = tensors[name].detach().contiguous().cpu()
            fh.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
