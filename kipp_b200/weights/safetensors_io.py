"""Writer for the safetensors container (the random-weights mode and tests
write model folders with it; the host core reads them, csrc/host/weights.hpp).

Layout: an 8-byte little-endian header length, a JSON header that maps each
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets
relative to the end of the header), then the raw little-endian tensor bytes.
A sharded checkpoint has ``model.safetensors.index.json`` whose ``weight_map``
names the shard file of each tensor.  The reference's converter reads the same
format (tools/convert_to_gguf.py:282-343).
"""
from __future__ import annotations

import json
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
