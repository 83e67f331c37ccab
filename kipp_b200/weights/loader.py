"""Checkpoint tensors by name: a face of the host core's reader
(csrc/host/weights.hpp), which maps the safetensors files of a model folder and
compares what they hold with what a model declares.

The reference binds 2 + 11*L (+1 untied) tensors by their exact name, type and
shape and fails on the first problem (src/kipp.c:859-1007, 1108-1118).  Here
all problems are collected and reported in one error: every missing tensor,
every unexpected one, every wrong shape and every unsupported dtype.

Storage dtype policy: 16-bit floats are kept as bfloat16 (float16 is converted
once), a tensor stored in 32-bit floats stays float32, integer tables become
int32.
"""
from __future__ import annotations

import ctypes
import json
from typing import Iterable

import numpy as np
import torch

from .. import native as N
from .spec import TensorSpec


class WeightError(ValueError):
    """Raised once with the complete list of problems of a checkpoint."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = [(n, tuple(a), tuple(b)) for n, a, b in wrong_shape]
        self.wrong_dtype = [(n, t) for n, t in wrong_dtype]
        super().__init__(message)

    @classmethod
    def from_message(cls, message: str) -> "WeightError":
        return cls(message)

    @classmethod
    def from_report(cls, report: dict) -> "WeightError":
        return cls(report["message"], report["missing"], report["unexpected"], report["wrong_shape"],
                   report["wrong_dtype"])


_TORCH = {N.DTYPE_F32: torch.float32, N.DTYPE_BF16: torch.bfloat16, N.DTYPE_F16: torch.float16,
          N.DTYPE_I32: torch.int32, N.DTYPE_I64: torch.int64, N.DTYPE_I16: torch.int16,
          N.DTYPE_I8: torch.int8, N.DTYPE_U8: torch.uint8}
_NUMPY = {N.DTYPE_F32: np.float32, N.DTYPE_BF16: np.int16, N.DTYPE_F16: np.float16, N.DTYPE_I32: np.int32,
          N.DTYPE_I64: np.int64, N.DTYPE_I16: np.int16, N.DTYPE_I8: np.int8, N.DTYPE_U8: np.uint8}


def storage_dtype(dtype: torch.dtype) -> torch.dtype | None:
    """The dtype a tensor stored as ``dtype`` is kept in, or None if unsupported."""
    if dtype in (torch.bfloat16, torch.float16):
        return torch.bfloat16
    if dtype == torch.float32:
        return torch.float32
    if dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    return None


def specs_json(specs: Iterable[TensorSpec]) -> bytes:
    return json.dumps([{"name": s.name, "shape": list(s.shape), "init": s.init, "optional": s.optional,
                        "alias_of": s.alias_of, "ignore_if_present": s.ignore_if_present}
                       for s in specs]).encode()


class Checkpoint:
    """The mapped safetensors files of a model folder."""

    def __init__(self, folder: str):
        self.folder = folder
        self._lib = N.lib()
        h = ctypes.c_void_p()
        N.check(self._lib.kipp_weights_open(folder.encode(), ctypes.byref(h)))
        self._h = h

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.kipp_weights_close(h)
            self._h = None

    def _info(self, name: str) -> N.TensorInfo:
        info = N.TensorInfo()
        N.check(self._lib.kipp_weights_find(self._h, name.encode(), ctypes.byref(info)))
        return info

    def names(self) -> list[str]:
        out = []
        info = N.TensorInfo()
        for i in range(self._lib.kipp_weights_count(self._h)):
            N.check(self._lib.kipp_weights_tensor(self._h, i, ctypes.byref(info)))
            out.append(info.name.decode())
        return out

    def __contains__(self, name: str) -> bool:
        info = N.TensorInfo()
        return self._lib.kipp_weights_find(self._h, name.encode(), ctypes.byref(info)) == 0

    def compare(self, specs: Iterable[TensorSpec]) -> dict:
        """What differs between the checkpoint and ``specs`` (lists of names and shapes)."""
        return json.loads(N.text_result(self._lib.kipp_weights_compare, self._h, specs_json(specs)))

    def check(self, specs: Iterable[TensorSpec]) -> None:
        report = self.compare(specs)
        if report["message"]:
            raise WeightError.from_report(report)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU copy of the tensor in the type it is stored in."""
        info = self._info(name)
        if info.dtype not in _TORCH:
            raise WeightError(f"tensor {name} has an element type the engine does not take")
        shape = tuple(info.shape[i] for i in range(info.ndim))
        count = int(np.prod(shape)) if shape else 1
        if info.bytes == 0:
            return torch.empty(shape, dtype=_TORCH[info.dtype])
        buf = (ctypes.c_char * info.bytes).from_address(info.data)
        arr = np.frombuffer(buf, dtype=_NUMPY[info.dtype], count=count).copy()
        t = torch.from_numpy(arr)
        if info.dtype == N.DTYPE_BF16:
            t = t.view(torch.bfloat16)
        return t.reshape(shape)


def open_checkpoint(folder: str) -> Checkpoint:
    return Checkpoint(folder)


def load_tensors(folder: str, specs: Iterable[TensorSpec]) -> dict[str, torch.Tensor]:
    """Read the tensors ``specs`` declares from ``folder`` as CPU tensors in
    their storage dtype.  Absent optional tensors are left out."""
    specs = list(specs)
    ckpt = Checkpoint(folder)
    ckpt.check(specs)
    out: dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name not in ckpt or (s.ignore_if_present and s.alias_of is not None):
            continue
        t = ckpt.tensor(s.name)
        out[s.name] = t.to(storage_dtype(t.dtype))
    return out
