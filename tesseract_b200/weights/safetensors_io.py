"""Reading and writing the safetensors container.

Layout: an 8-byte little-endian header length, a JSON header that maps each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian tensor bytes.
The reference opens the same container through a crate and validates dtype,
shape and byte length per tensor (src/model/weights.rs:181-275); this reader
does the same by hand and supports a sharded folder through
``model.safetensors.index.json`` (src/model/weights.rs:181-229).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The container itself is malformed (not a statement about a model)."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int
    shard: int


class SafetensorsFile:
    """One memory-mapped ``.safetensors`` file; tensors are views of the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._handle = open(path, "rb")
        except OSError as exc:
            raise SafetensorsError(f"{path}: cannot open: {exc}") from exc
        size = os.fstat(self._handle.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        (header_len,) = struct.unpack("<Q", self._handle.read(8))
        if header_len > size - 8:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._handle.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON: {exc}") from exc
        self._data_start = 8 + header_len
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_COPY)
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        data_len = size - self._data_start
        for name, info in header.items():
            try:
                dtype_name = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as exc:
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from exc
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype_name}")
            dtype, width = _DTYPES[dtype_name]
            count = 1
            for s in shape:
                count *= s
            if not (0 <= begin <= end <= data_len) or end - begin != count * width:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' byte range [{begin},{end}) does not match shape {list(shape)} {dtype_name}"
                )
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, 0)

    def names(self) -> List[str]:
        return sorted(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        entry = self.entries[name]
        count = 1
        for s in entry.shape:
            count *= s
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        flat = torch.frombuffer(self._map, dtype=entry.dtype, count=count,
                                offset=self._data_start + entry.begin)
        return flat.view(entry.shape)


class SafetensorsSource:
    """All tensors of a model folder, looked up by name."""

    SINGLE = "model.safetensors"
    INDEX = "model.safetensors.index.json"

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, self.SINGLE)
        index = os.path.join(model_dir, self.INDEX)
        self._files: List[SafetensorsFile] = []
        self._where: Dict[str, int] = {}
        if os.path.exists(single):
            self._files.append(SafetensorsFile(single))
            for name in self._files[0].entries:
                self._where[name] = 0
        elif os.path.exists(index):
            with open(index, "r", encoding="utf-8") as handle:
                try:
                    weight_map = json.load(handle)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError) as exc:
                    raise SafetensorsError(f"{index}: no usable 'weight_map'") from exc
            shards: Dict[str, int] = {}
            for name, shard_name in weight_map.items():
                if shard_name not in shards:
                    shards[shard_name] = len(self._files)
                    self._files.append(SafetensorsFile(os.path.join(model_dir, shard_name)))
                shard = shards[shard_name]
                if name not in self._files[shard].entries:
                    raise SafetensorsError(f"{index}: tensor '{name}' is not in shard {shard_name}")
                self._where[name] = shard
        else:
            raise SafetensorsError(f"{model_dir}: neither {self.SINGLE} nor {self.INDEX} exists")

    def names(self) -> List[str]:
        return sorted(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def entry(self, name: str) -> TensorEntry:
        return self._files[self._where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write ``tensors`` (CPU, contiguous) as one safetensors file, names sorted."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        tensor = tensors[name].detach().cpu().contiguous()
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {tensor.dtype}, which safetensors cannot hold")
        raw = tensor.reshape(-1).view(torch.uint8).numpy().tobytes() if tensor.numel() else b""
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for raw in blobs:
            handle.write(raw)
