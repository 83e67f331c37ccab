"""Dense SwiGLU feed-forward: x += W_down (silu(W_gate n) * (W_up n))
(src/kipp.c:2994-3010, silu src/kipp.c:2402-2404).  The part itself:
csrc/host/parts.hpp."""
from __future__ import annotations

from .base import FeedForward


class SwiGLUFeedForward(FeedForward):
    kind = "swiglu"

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}
