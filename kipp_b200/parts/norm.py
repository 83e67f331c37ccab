"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, computed in float32
(src/kipp.c:2221-2231).  The part itself: csrc/host/parts.hpp."""
from __future__ import annotations

from .base import Norm


class RMSNorm(Norm):
    kind = "rmsnorm"

    def __init__(self, size: int, eps: float, weight_name: str = "weight"):
        self.size = size
        self.eps = float(eps)
        self.weight_name = weight_name

    def params(self, prefix, ctx) -> dict:
        return {"size": self.size, "eps": self.eps, "weight_name": self.weight_name}
