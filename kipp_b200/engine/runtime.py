"""What the parts need at run time: device, compute dtype, kernels, activation
workspace and the device status word."""
from __future__ import annotations

import torch

from .. import kernels


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.float32, torch.bfloat16):
            return name
        raise ValueError(f"compute dtype must be float32 or bfloat16, not {name}")
    table = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
             "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
    try:
        return table[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}; use bfloat16 or float32") from None


class Workspace:
    """Named activation buffers that grow to the largest size asked for and are
    then reused by every step (one workspace per engine, not per request, as
    the reference's Metal bridge keeps it, src/metal/kipp_metal.m:151-158)."""

    def __init__(self, device: torch.device):
        self.device = device
        self._flat: dict[tuple[str, torch.dtype], torch.Tensor] = {}
        self.generation = 0          # bumped whenever a buffer moves (captured graphs go stale)

    def buffer(self, key: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        flat = self._flat.get((key, dtype))
        if flat is None or flat.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace buffer {key!r} would be allocated inside a graph capture")
            flat = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._flat[(key, dtype)] = flat
            self.generation += 1
        return flat[:n].view(shape)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())


class Runtime:
    def __init__(self, device: str | torch.device = "cuda:0", dtype="bfloat16"):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("kipp_b200 runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; kipp_b200 has no CPU fallback")
        self.dtype = parse_dtype(dtype)
        self.ops = kernels
        self.workspace = Workspace(self.device)
        # Kernels record refused accesses here (1 token id out of range, 2 write
        # to an unmapped page, 3 read of an unmapped page) instead of faulting.
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)

    def check_status(self) -> None:
        code = int(self.status[0].item())
        if code:
            self.status.zero_()
            what = {1: "a token id outside the vocabulary",
                    2: "a write to an unmapped cache page",
                    3: "a read of an unmapped cache page"}.get(code, f"code {code}")
            raise RuntimeError(f"a kernel refused {what}")
