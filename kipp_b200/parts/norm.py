"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, computed in float32
(src/kipp.c:2221-2231)."""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.spec import INIT_NEAR_ONE, TensorSpec
from .base import Norm


class RMSNorm(Norm):
    def __init__(self, size: int, eps: float, weight_name: str = "weight"):
        self.size = size
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + self.weight_name, (self.size,), INIT_NEAR_ONE)]

    def bind(self, tensors, prefix, runtime) -> None:
        # The scale keeps its storage dtype (bfloat16 or float32).
        self.weight = tensors[prefix + self.weight_name].to(runtime.device).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx, x, rows=None, n_rows=None, key="normed"):
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = ctx.workspace.buffer(key, (n, self.size), ctx.dtype)
        ctx.ops.rmsnorm(out, x, self.weight, self.eps, rows, n)
        return out
