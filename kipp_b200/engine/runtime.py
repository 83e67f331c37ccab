"""Compute dtypes by name."""
from __future__ import annotations

import torch


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
