"""Reading and writing the safetensors container, without a library.

The format: 8 bytes little-endian header length ``n``; ``n`` bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": ...}``;
then the raw little-endian tensor bytes, offsets relative to the end of the
header.  A model folder holds either ``model.safetensors`` or a
``model.safetensors.index.json`` whose ``weight_map`` names shard files (the
reference resolves both the same way, ``models/loader.py:140-151,188-215``).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Iterable, Mapping

import torch

_DTYPES: dict[str, torch.dtype] = {
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


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int
    file: str


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are read on demand."""

    def __init__(self, path: str) -> None:
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file")
        try:
            header = json.loads(self._fh.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self._data_start = 8 + n
        self.metadata = header.pop("__metadata__", None) or {}
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
            except KeyError:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has unsupported dtype {info.get('dtype')!r}"
                ) from None
            begin, end = info["data_offsets"]
            shape = tuple(int(s) for s in info["shape"])
            numel = 1
            for s in shape:
                numel *= s
            if end - begin != numel * _itemsize(dtype) or self._data_start + end > size:
                raise SafetensorsError(f"{path}: tensor {name!r} has inconsistent offsets")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, path)
        self._mm = (
            mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None
        )

    def names(self) -> list[str]:
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns a copy of the bytes (safe after ``close``)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        raw = memoryview(self._mm)[self._data_start + e.begin : self._data_start + e.end]
        flat = torch.frombuffer(raw, dtype=e.dtype).clone()
        return flat.reshape(e.shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None
        self._fh.close()


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class Checkpoint:
    """All tensors of a model folder, over one file or an index of shards."""

    def __init__(self, model_dir: str) -> None:
        self.model_dir = os.fspath(model_dir)
        index = os.path.join(self.model_dir, "model.safetensors.index.json")
        single = os.path.join(self.model_dir, "model.safetensors")
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f)["weight_map"]
            files = sorted(set(weight_map.values()))
        elif os.path.isfile(single):
            files = ["model.safetensors"]
        else:
            raise FileNotFoundError(
                f"{self.model_dir!r} holds neither model.safetensors nor "
                "model.safetensors.index.json"
            )
        self._files = [SafetensorsFile(os.path.join(self.model_dir, f)) for f in files]
        self.entries: dict[str, TensorEntry] = {}
        self._owner: dict[str, SafetensorsFile] = {}
        for sf in self._files:
            for name, e in sf.entries.items():
                self.entries[name] = e
                self._owner[name] = sf

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name].shape

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name].dtype

    def read(self, name: str) -> torch.Tensor:
        return self._owner[name].read(name)

    def close(self) -> None:
        for sf in self._files:
            sf.close()

    def __enter__(self) -> "Checkpoint":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def write_safetensors(
    path: str,
    tensors: Mapping[str, torch.Tensor] | Iterable[tuple[str, torch.Tensor]],
    metadata: Mapping[str, str] | None = None,
) -> None:
    """Write tensors (CPU, any supported dtype) as one safetensors file."""
    items = list(tensors.items()) if isinstance(tensors, Mapping) else list(tensors)
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs: list[torch.Tensor] = []
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        t = t.detach().to("cpu").contiguous()
        nbytes = t.numel() * t.element_size()
        header[name] = {
            "dtype": _NAMES[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
        blobs.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((-len(raw)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
