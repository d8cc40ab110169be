"""Reading and writing the safetensors container without any helper package.

Layout: 8 bytes little-endian header length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the raw little-endian tensor bytes.  The file is memory-mapped; a tensor is read by
name and only its bytes are touched (the reference maps ``model.safetensors`` the same
way, src/model/falconh1_loader.cpp:17-22).  A folder may also hold
``model.safetensors.index.json`` with a ``weight_map`` from names to shard files.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped file: ``keys()``, ``info(name)`` -> (dtype name, shape), ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as exc:
            raise SafetensorsError(f"cannot open {path}: {exc}") from exc
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not JSON: {exc}") from exc
        self.metadata = header.pop("__metadata__", {}) or {}
        self._entries: Dict[str, dict] = header
        self._data_start = 8 + hlen
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        data_len = size - self._data_start
        for name, ent in self._entries.items():
            if ent.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unknown dtype {ent.get('dtype')}")
            b, e = ent["data_offsets"]
            numel = 1
            for s in ent["shape"]:
                numel *= int(s)
            if not (0 <= b <= e <= data_len) or e - b != numel * _DTYPES[ent["dtype"]][1]:
                raise SafetensorsError(f"{path}: tensor byte size mismatch for {name}")

    def keys(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        ent = self._entries[name]
        return ent["dtype"], tuple(int(s) for s in ent["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns a copy of the bytes."""
        ent = self._entries[name]
        dtype, _ = _DTYPES[ent["dtype"]]
        b, e = ent["data_offsets"]
        shape = tuple(int(s) for s in ent["shape"])
        if e == b:
            return torch.empty(shape, dtype=dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=e - b, offset=self._data_start + b)
        return torch.from_numpy(raw.copy()).view(dtype).reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        finally:
            self._fh.close()


class ModelFiles:
    """All tensors of a model folder: the single ``model.safetensors`` or the shards of an index."""

    def __init__(self, model_dir: str):
        self.files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as fh:
                weight_map = json.load(fh).get("weight_map", {})
            paths = [os.path.join(model_dir, p) for p in sorted(set(weight_map.values()))]
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                                   "model.safetensors.index.json found")
        for p in paths:
            f = SafetensorsFile(p)
            self.files.append(f)
            for k in f.keys():
                self._where[k] = f

    def keys(self) -> List[str]:
        return list(self._where)

    def info(self, name: str):
        return self._where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Mapping[str, str] = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) as one safetensors file, names sorted."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs: List[bytes] = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(hjson)))
        fh.write(hjson)
        for raw in blobs:
            fh.write(raw)
    os.replace(tmp, path)
