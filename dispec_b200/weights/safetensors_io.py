"""Reader and writer of the safetensors container, by tensor name.

Format: 8 bytes little-endian header length N, N bytes of JSON
(``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``), then the
raw little-endian tensor bytes; offsets are relative to the end of the header.  A model
folder holds ``model.safetensors`` or shards listed in ``model.safetensors.index.json``
(``weight_map``: name -> file).  The reference leaves this to a library call
(puneethgv/DiSpec dispec/models/loader.py:18-27).
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if 8 + n > size:
            raise SafetensorsError(f"{path}: truncated (header of {n} bytes, file of {size})")
        try:
            header = json.loads(self._f.read(n))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries = header
        self._data_start = 8 + n
        self._size = size
        # private copy-on-write mapping: tensors over it are writable without touching the file
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None
        for name, e in header.items():
            if e["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {e['dtype']}")
            b, end = e["data_offsets"]
            if self._data_start + end > size or b > end:
                raise SafetensorsError(f"{path}: tensor {name!r} lies outside the file (truncated?)")

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def get(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dtype = _DTYPES[e["dtype"]]
        b, end = e["data_offsets"]
        shape = tuple(e["shape"])
        count = 1
        for s in shape:
            count *= s
        if count * torch.empty((), dtype=dtype).element_size() != end - b:
            raise SafetensorsError(f"{self.path}: tensor {name!r}: {end - b} bytes for shape {shape}")
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        t = torch.frombuffer(self._mm, dtype=dtype, count=count, offset=self._data_start + b)
        return t.reshape(shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive; only the descriptor is closed here
        self._f.close()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        ordered.append(t)
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for t in ordered:
            if t.numel():
                f.write(memoryview(t.view(torch.uint8).reshape(-1).numpy()))


class CheckpointFolder:
    """All tensors of a model folder, single file or shards."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self._files: dict[str, SafetensorsFile] = {}
        self._where: dict[str, str] = {}
        if os.path.exists(index):
            with open(index) as f:
                weight_map = json.load(f)["weight_map"]
            for name, fname in weight_map.items():
                self._where[name] = fname
            for fname in sorted(set(weight_map.values())):
                path = os.path.join(folder, fname)
                if not os.path.exists(path):
                    raise SafetensorsError(f"{index} names {fname}, which is missing")
                self._files[fname] = SafetensorsFile(path)
                for name in self._files[fname].names():
                    self._where.setdefault(name, fname)
        elif os.path.exists(single):
            self._files["model.safetensors"] = SafetensorsFile(single)
            for name in self._files["model.safetensors"].names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> list[str]:
        return list(self._where)

    def shape(self, name: str):
        return self._files[self._where[name]].shape(name)

    def dtype(self, name: str):
        return self._files[self._where[name]].dtype(name)

    def get(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].get(name)
