"""Reading and writing safetensors files.

The format: eight bytes of little-endian header length, a JSON header that maps
each tensor name to ``{"dtype", "shape", "data_offsets"}``, then the tensors'
bytes.  The reference loads every tensor of every shard into a map by name
(src/weights.rs:22-63); this reader does the same through a memory map, so that
a tensor's bytes are touched only when it is asked for.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple
    begin: int
    end: int
    file: "SafetensorsFile"

    def load(self) -> torch.Tensor:
        return self.file.tensor(self.name)


class SafetensorsFile:
    """One safetensors file, opened read-only; ``entries`` maps names to ``TensorEntry``."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._fh.read(hlen))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {})
        self._data_start = 8 + hlen
        self._map = None
        self.entries = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            begin, end = info["data_offsets"]
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(info["shape"])
            count = 1
            for d in shape:
                count *= d
            if end - begin != count * dtype.itemsize or self._data_start + end > size:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, self)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if self._map is None:
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._map)[self._data_start + e.begin:self._data_start + e.end]
        # frombuffer shares the read-only map; clone so the caller owns writable memory
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=e.dtype)
        return t.reshape(e.shape).clone()


def save_file(tensors: dict, path: str, metadata: dict | None = None) -> None:
    """Write ``tensors`` (name -> CPU tensor) as one safetensors file, names sorted."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            fh.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def open_model_files(folder: str) -> list:
    """The safetensors files of a model folder, as the reference picks them
    (src/weights.rs:25-43): the shard names of ``model.safetensors.index.json`` if it
    exists, else every ``*.safetensors`` in the folder; sorted, without duplicates."""
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as fh:
            weight_map = json.load(fh).get("weight_map")
        if not isinstance(weight_map, dict):
            raise SafetensorsError(f"{index}: missing weight_map")
        names = sorted(set(weight_map.values()))
    else:
        names = sorted(n for n in os.listdir(folder) if n.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"no safetensors in {folder}")
    return [SafetensorsFile(os.path.join(folder, n)) for n in names]
