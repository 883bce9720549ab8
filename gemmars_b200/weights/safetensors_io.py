"""Reading and writing safetensors files, and a model folder's tensors by name.

File format (src/safetensors.rs:228-235, 272-317): an 8-byte little-endian header length, a
JSON header ``{name: {dtype, shape, data_offsets}}`` (plus ``__metadata__``), then the data;
offsets are relative to the end of the header.  A folder holds ``model.safetensors`` or
``model.safetensors.index.json`` whose ``weight_map`` names the shard of each tensor
(src/safetensors.rs:502-529).

Tensors are returned in the precision they are stored in: BF16 stays bfloat16, F32 stays
float32, F16 is widened (exactly) to float32, integer tables become int32.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Optional, Tuple

import torch


class WeightFileError(ValueError):
    pass


_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def kept_dtype(stored: torch.dtype) -> torch.dtype:
    """The precision a stored tensor is held in after loading."""
    if stored in (torch.bfloat16, torch.float32):
        return stored
    if stored in (torch.float16, torch.float64):
        return torch.float32
    return torch.int32


class SafetensorsFile:
    """One mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightFileError(f"{path}: {e.strerror}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise WeightFileError(f"{path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if 8 + hlen > size:
            raise WeightFileError(f"{path}: header length {hlen} exceeds file")  # src/safetensors.rs:229-231
        try:
            header = json.loads(self._f.read(hlen))
        except json.JSONDecodeError as e:
            raise WeightFileError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        # a private copy-on-write mapping: torch wants a writable buffer, the file is never written
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        self._info: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, inf in header.items():
            if inf["dtype"] not in _DTYPES:
                raise WeightFileError(f"{path}: tensor {name} has unsupported dtype {inf['dtype']}")
            dt, width = _DTYPES[inf["dtype"]]
            shape = tuple(int(s) for s in inf["shape"])
            lo, hi = inf["data_offsets"]
            n = 1
            for s in shape:
                n *= s
            if hi - lo != n * width or self._base + hi > size or lo < 0:
                raise WeightFileError(f"{path}: tensor {name} out of bounds")  # src/safetensors.rs:298-300
            self._info[name] = (dt, shape, self._base + lo, self._base + hi)

    def names(self) -> Iterable[str]:
        return self._info.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self._info[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor's stored bytes as a CPU tensor over the mapping (no copy)."""
        dt, shape, lo, hi = self._info[name]
        if hi == lo:
            return torch.empty(shape, dtype=dt)
        flat = torch.frombuffer(self._map, dtype=dt, count=(hi - lo) // _DTYPES[_NAMES[dt]][1], offset=lo)
        return flat.view(shape)


class ModelFiles:
    """The tensors of a model folder, by name, over one file or several shards."""

    def __init__(self, folder: str):
        self.folder = folder
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        self._shards: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, SafetensorsFile] = {}
        if os.path.exists(single):
            f = SafetensorsFile(single)
            self._shards[single] = f
            for n in f.names():
                self._where[n] = f
        elif os.path.exists(index):
            with open(index) as fh:
                weight_map = json.load(fh).get("weight_map", {})
            for n, shard in weight_map.items():
                path = os.path.join(folder, shard)
                if path not in self._shards:
                    self._shards[path] = SafetensorsFile(path)
                if n not in set(self._shards[path].names()):
                    raise WeightFileError(f"{index}: tensor {n} is not in {shard}")
                self._where[n] = self._shards[path]
        else:
            raise WeightFileError(f"{folder}: no model.safetensors or model.safetensors.index.json found")

    def names(self) -> set:
        return set(self._where)

    def has(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str):
        return self._where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None) -> None:
    """Writes ``tensors`` (CPU or device, any listed dtype) as one safetensors file."""
    header, offset, order = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightFileError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
        order.append(name)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
