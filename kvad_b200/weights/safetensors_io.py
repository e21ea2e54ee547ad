"""Reading and writing safetensors files without a helper library.

The format is small: eight bytes of little-endian header length, a JSON
header `{name: {dtype, shape, data_offsets}}`, then one blob that the offsets
index (bisand/kvad describes it at crates/llm/src/weights.rs:9-13 and writes
it at crates/nervus/src/checkpoint.rs:101-131, header padded with spaces to a
multiple of eight).  A model folder holds either `model.safetensors` or the
shards that `model.safetensors.index.json` names
(crates/llm/src/weights.rs:231-239, 269-282).

Files are memory-mapped; a tensor's bytes are touched only when it is read.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Iterable

import numpy as np
import torch

# safetensors dtype string -> (torch dtype, numpy carrier dtype, bytes per element)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I16": (torch.int16, np.dtype("<i2"), 2),
    "I8": (torch.int8, np.dtype("i1"), 1),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_TORCH_TO_NAME = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                 # safetensors spelling: "F32", "BF16", ...
    shape: tuple[int, ...]
    file: str
    begin: int                 # absolute byte offset in `file`
    end: int

    @property
    def is_float(self) -> bool:
        return self.dtype in ("F32", "BF16", "F16", "F64")

    @property
    def is_int(self) -> bool:
        return self.dtype in ("I64", "I32", "I16", "I8", "U8")


def _read_header(path: str) -> tuple[dict, int]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", raw)
        if n > size - 8 or n > (1 << 31):
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    return header, 8 + n


class Checkpoint:
    """Every tensor of a model folder, by name, over one or several files."""

    def __init__(self, files: Iterable[str]):
        self.entries: dict[str, TensorEntry] = {}
        self._maps: dict[str, mmap.mmap] = {}
        self._handles = []
        for path in files:
            header, base = _read_header(path)
            size = os.path.getsize(path)
            for name, info in header.items():
                if name == "__metadata__":
                    continue
                try:
                    dtype = str(info["dtype"])
                    shape = tuple(int(s) for s in info["shape"])
                    lo, hi = (int(x) for x in info["data_offsets"])
                except (KeyError, TypeError, ValueError):
                    raise SafetensorsError(f"{path}: malformed header entry for `{name}`") from None
                if dtype not in _DTYPES:
                    raise SafetensorsError(f"{path}: tensor `{name}` has dtype {dtype}, which this library does not read")
                want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][2] if shape else _DTYPES[dtype][2]
                if hi - lo != want or base + hi > size or lo < 0:
                    raise SafetensorsError(
                        f"{path}: tensor `{name}` {dtype}{list(shape)} needs {want} bytes but its offsets span {hi - lo}")
                if name in self.entries:
                    raise SafetensorsError(f"tensor `{name}` is in both {self.entries[name].file} and {path}")
                self.entries[name] = TensorEntry(name, dtype, shape, path, base + lo, base + hi)

    @classmethod
    def open_dir(cls, model_dir: str) -> "Checkpoint":
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(single):
            return cls([single])
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            shards = sorted({os.path.join(model_dir, v) for v in weight_map.values()})
            if not shards:
                raise SafetensorsError(f"{index}: weight_map names no file")
            return cls(shards)
        raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> list[str]:
        return sorted(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def _map(self, path: str) -> mmap.mmap:
        m = self._maps.get(path)
        if m is None:
            f = open(path, "rb")
            self._handles.append(f)
            m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[path] = m
        return m

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (a CPU tensor that owns its memory)."""
        e = self.entries[name]
        tdt, ndt, _ = _DTYPES[e.dtype]
        count = int(np.prod(e.shape, dtype=np.int64)) if e.shape else 1
        arr = np.frombuffer(self._map(e.file), dtype=ndt, count=count, offset=e.begin).copy()
        t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif tdt == torch.bool:
            t = t.to(torch.bool)
        return t.reshape(e.shape)

    def close(self) -> None:
        for m in self._maps.values():
            m.close()
        for f in self._handles:
            f.close()
        self._maps.clear()
        self._handles.clear()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Writes `tensors` (CPU, contiguous) in name order, atomically."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot store `{name}` of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".partial"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            elif t.dtype == torch.bool:
                t = t.to(torch.uint8)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
