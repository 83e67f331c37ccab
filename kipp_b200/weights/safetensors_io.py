"""Reader and writer for the safetensors container.

Layout: an 8-byte little-endian header length, a JSON header that maps each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian tensor bytes.
A sharded checkpoint has ``model.safetensors.index.json`` whose ``weight_map``
names the shard file of each tensor.  The reference's converter reads the same
format (tools/convert_to_gguf.py:282-343).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterable

import torch

_DTYPES = {
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F32": torch.float32,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


def _element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class SafetensorsFile:
    """One mapped safetensors file; tensors are views of the mapping."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{path}: truncated safetensors header")
            (hlen,) = struct.unpack("<Q", head)
            if hlen > _MAX_HEADER or 8 + hlen > size:
                raise SafetensorsError(f"{path}: unreasonable safetensors header length {hlen}")
            try:
                header = json.loads(f.read(hlen))
            except (json.JSONDecodeError, UnicodeDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
            self._data_start = 8 + hlen
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY) if size else None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        data_size = size - self._data_start
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(d) for d in info["shape"])
                begin, end = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: bad header entry for {name!r}: {info!r}") from None
            count = 1
            for d in shape:
                count *= d
            if begin < 0 or end < begin or end > data_size or end - begin != count * _element_size(dtype):
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has byte range [{begin}, {end}) that does not fit "
                    f"{info['dtype']} {list(shape)} in a data section of {data_size} bytes")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self) -> list[str]:
        return list(self.entries)

    def info(self, name: str) -> tuple[torch.dtype, tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the mapped bytes (clone before writing)."""
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        count = (end - begin) // _element_size(dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=count,
                                offset=self._data_start + begin)
        return flat.view(shape)


def open_checkpoint(folder: str) -> dict[str, tuple[SafetensorsFile, str]]:
    """Map tensor name -> (file, name) over all shards of a model folder."""
    index_path = os.path.join(folder, "model.safetensors.index.json")
    files: dict[str, SafetensorsFile] = {}
    out: dict[str, tuple[SafetensorsFile, str]] = {}
    if os.path.isfile(index_path):
        with open(index_path, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map")
        if not isinstance(weight_map, dict):
            raise SafetensorsError(f"{index_path}: no weight_map")
        for name, shard in weight_map.items():
            if shard not in files:
                path = os.path.join(folder, shard)
                if not os.path.isfile(path):
                    raise SafetensorsError(f"{index_path} names shard {shard!r}, which is absent")
                files[shard] = SafetensorsFile(path)
            if name not in files[shard].entries:
                raise SafetensorsError(f"{shard}: index lists tensor {name!r} but the file lacks it")
            out[name] = (files[shard], name)
        return out
    single = os.path.join(folder, "model.safetensors")
    if not os.path.isfile(single):
        raise SafetensorsError(
            f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
    file = SafetensorsFile(single)
    return {name: (file, name) for name in file.names()}


def write_safetensors(path: str, tensors: Iterable[tuple[str, torch.Tensor]],
                      metadata: dict[str, str] | None = None) -> None:
    """Write ``(name, tensor)`` pairs; each tensor's bytes start 64-byte aligned
    relative to the file start so that mapped views are aligned."""
    items = [(name, t.detach().cpu().contiguous()) for name, t in tensors]
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    ranges = []
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        ranges.append((offset, nbytes))
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (-(8 + len(blob))) % 64
    blob += b" " * pad
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for (name, t), (_, nbytes) in zip(items, ranges):
            if nbytes:
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
