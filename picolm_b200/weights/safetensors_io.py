"""A small reader and writer of the safetensors container.

Format (as the reference's vendored reader parses it, picolm/csafetensors.h:49-79):
an 8-byte little-endian header length, a JSON object
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}` (plus an optional
`__metadata__`), then the raw little-endian tensor bytes.  A sharded checkpoint
has `model.safetensors.index.json` whose `weight_map` names the file of every
tensor (the reference guesses shard names instead, picolm/safetensors.c:213-227).
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
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                 # the container's dtype string, e.g. "BF16"
    shape: Tuple[int, ...]
    file: str
    begin: int                 # byte offsets inside the file
    end: int


class SafetensorsFile:
    """One mmap'd file; `tensor(name)` returns a CPU tensor that views the map."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file of {size} bytes")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", None) or {}
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        base = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            b, e = info["data_offsets"]
            shape = tuple(int(s) for s in info["shape"])
            dt = info["dtype"]
            if base + e > size or b > e:
                raise SafetensorsError(f"{path}: tensor {name!r} lies outside the file")
            if dt in _DTYPES:
                n = 1
                for s in shape:
                    n *= s
                if n * _DTYPES[dt].itemsize != e - b:
                    raise SafetensorsError(
                        f"{path}: tensor {name!r} has {e - b} bytes, its shape {list(shape)} of {dt} needs "
                        f"{n * _DTYPES[dt].itemsize}")
            self.entries[name] = TensorEntry(name, dt, shape, path, base + b, base + e)

    def tensor(self, name: str) -> torch.Tensor:
        ent = self.entries[name]
        if ent.dtype not in _DTYPES:
            raise SafetensorsError(f"{self.path}: tensor {name!r} has the unsupported dtype {ent.dtype}")
        dtype = _DTYPES[ent.dtype]
        count = (ent.end - ent.begin) // dtype.itemsize
        if count == 0:
            return torch.empty(ent.shape, dtype=dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=ent.begin)
        return flat.reshape(ent.shape)

    def close(self) -> None:
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass                    # tensors still view the map; it closes with them
        self._f.close()


class Checkpoint:
    """All tensors of a model folder, by name, across shards."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        files: List[str]
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f)["weight_map"]
            files = sorted(set(weight_map.values()))
        elif os.path.exists(single):
            files = ["model.safetensors"]
        else:
            raise FileNotFoundError(
                f"{model_dir}: neither model.safetensors nor model.safetensors.index.json is there")
        self.files = [SafetensorsFile(os.path.join(model_dir, f)) for f in files]
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for sf in self.files:
            for name, ent in sf.entries.items():
                self.entries[name] = ent
                self._owner[name] = sf

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    def close(self) -> None:
        for sf in self.files:
            sf.close()


def save_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write CPU tensors to one file without gaps: wider element types first, then
    by name, so that every tensor starts on a multiple of its element size."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors, key=lambda n: (-tensors[n].element_size(), n))
    blobs = []
    for name in order:
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
