"""Bind checkpoint tensors to the names a model declares.

The reference binds 2 + 11*L (+1 untied) tensors by their exact name, type and
shape and fails on the first problem (src/kipp.c:859-1007, 1108-1118).  Here
all problems are collected and reported in one error: every missing tensor,
every unexpected one, every wrong shape and every unsupported dtype.

Storage dtype policy: 16-bit floats are kept as bfloat16 (float16 is converted
once), a tensor stored in 32-bit floats stays float32, integer tables become
int32.
"""
from __future__ import annotations

from typing import Iterable, Mapping

import torch

from .safetensors_io import SafetensorsError, open_checkpoint
from .spec import TensorSpec


class WeightError(ValueError):
    """Raised once with the complete list of problems of a checkpoint."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, where=""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"checkpoint {where} does not match the model:" if where
                 else "checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  unsupported dtype: {name} is {got}")
        super().__init__("\n".join(lines))


def storage_dtype(dtype: torch.dtype) -> torch.dtype | None:
    """The dtype a tensor stored as ``dtype`` is kept in, or None if unsupported."""
    if dtype in (torch.bfloat16, torch.float16):
        return torch.bfloat16
    if dtype == torch.float32:
        return torch.float32
    if dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    return None


def check_tensors(specs: Iterable[TensorSpec],
                  available: Mapping[str, tuple[torch.dtype, tuple[int, ...]]],
                  where: str = "") -> None:
    """Compare declared tensors with ``name -> (dtype, shape)``; raise WeightError
    listing every difference."""
    specs = list(specs)
    declared = {s.name for s in specs}
    missing, wrong_shape, wrong_dtype = [], [], []
    for s in specs:
        if s.name not in available:
            if s.optional and (s.alias_of is None or s.alias_of in available):
                continue
            missing.append(s.name)
            continue
        dtype, shape = available[s.name]
        if tuple(shape) != tuple(s.shape):
            wrong_shape.append((s.name, tuple(shape), tuple(s.shape)))
        if storage_dtype(dtype) is None:
            wrong_dtype.append((s.name, str(dtype)))
    unexpected = sorted(n for n in available if n not in declared)
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype, where)


def load_tensors(folder: str, specs: Iterable[TensorSpec]) -> dict[str, torch.Tensor]:
    """Read the tensors ``specs`` declares from ``folder`` as CPU tensors in
    their storage dtype.  Absent optional tensors are left out."""
    specs = list(specs)
    try:
        table = open_checkpoint(folder)
    except SafetensorsError as e:
        raise WeightError([], [], [], [], where=f"{folder} ({e})") from None
    available = {name: file.info(key) for name, (file, key) in table.items()}
    ignored = {s.name for s in specs if s.ignore_if_present}
    check_tensors(specs, available, where=folder)
    out: dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name not in table or s.name in ignored and s.alias_of is not None:
            continue
        file, key = table[s.name]
        t = file.tensor(key)
        out[s.name] = t.to(storage_dtype(t.dtype))
    return out
