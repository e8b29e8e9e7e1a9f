"""Reading and writing safetensors files without a helper package.

The format is an 8-byte little-endian header length, a JSON header mapping
tensor name -> ``{"dtype", "shape", "data_offsets"}``, then the raw bytes.  The
reference reads the same header by hand when it only needs metadata
(python/freetoken/models/weight.py:98-104) and finds shards through
``model.safetensors.index.json`` or a folder scan
(python/freetoken/models/minimax_m3/weight.py:66-97,
python/freetoken/models/loader.py:168-175).
"""

from __future__ import annotations

import glob
import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
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
    """Where one tensor lives: file, dtype, shape and byte range."""

    name: str
    path: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are read on demand."""

    def __init__(self, path: str):
        self.path = path
        self._file = open(path, "rb")
        head = self._file.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: too short to be a safetensors file")
        (header_len,) = struct.unpack("<Q", head)
        header = json.loads(self._file.read(header_len))
        self._data_start = 8 + header_len
        self._map = None
        self.entries: Dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dtype = _DTYPES.get(meta["dtype"])
            if dtype is None:
                raise ValueError(f"{path}: tensor '{name}' has unsupported dtype {meta['dtype']}")
            begin, end = meta["data_offsets"]
            self.entries[name] = TensorEntry(name, path, dtype, tuple(meta["shape"]), begin, end)

    def read(self, name: str) -> torch.Tensor:
        entry = self.entries[name]
        if self._map is None:
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        count = 1
        for s in entry.shape:
            count *= s
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        with warnings.catch_warnings():
            # the mapping is read-only; the tensor is copied before anyone can write to it
            warnings.simplefilter("ignore", UserWarning)
            flat = torch.frombuffer(
                self._map, dtype=entry.dtype, count=count, offset=self._data_start + entry.begin
            )
        return flat.reshape(entry.shape).clone()

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._file.close()


class Checkpoint:
    """All tensors of a model folder, by name, whichever shard holds them."""

    def __init__(self, folder: str):
        self.folder = folder
        paths = _shard_paths(folder)
        if not paths:
            raise FileNotFoundError(f"{folder}: no .safetensors file found")
        self._files: List[SafetensorsFile] = [SafetensorsFile(p) for p in paths]
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for f in self._files:
            for name, entry in f.entries.items():
                self.entries[name] = entry
                self._owner[name] = f

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def read(self, name: str) -> torch.Tensor:
        return self._owner[name].read(name)

    def close(self) -> None:
        for f in self._files:
            f.close()

    def __enter__(self) -> "Checkpoint":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def _shard_paths(folder: str) -> List[str]:
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        return [os.path.join(folder, p) for p in sorted(set(weight_map.values()))]
    single = os.path.join(folder, "model.safetensors")
    if os.path.exists(single):
        return [single]
    return sorted(glob.glob(os.path.join(folder, "*.safetensors")))


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write ``tensors`` (CPU or device) to one file, names in sorted order."""
    header: Dict[str, dict] = {}
    offset = 0
    ordered = sorted(tensors.items())
    for name, t in ordered:
        if t.dtype not in _NAMES:
            raise ValueError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {
            "dtype": _NAMES[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in ordered:
            c = t.detach().contiguous().cpu()
            f.write(c.reshape(-1).view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    os.replace(tmp, path)
