"""Causal grouped-query attention over the paged cache, with optional per-head
q/k RMSNorm and a position encoding applied to q and k.

Order of operations as the reference's block (docs/ARCHITECTURE.md:77-92,
src/kipp.c:2950-2993): q/k/v projections (no bias) -> per-head norm of q and k
-> rotation -> keys and values into the cache -> attention -> output
projection added to the residual stream.  The part itself: csrc/host/parts.hpp.
"""
from __future__ import annotations

from typing import Optional

from .base import Mixer, PagedKVSpec, PositionEncoding


class AttentionMixer(Mixer):
    kind = "attention"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PositionEncoding, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = scale
        self.q_dim = num_heads * head_dim
        self.kv_dim = num_kv_heads * head_dim

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads,
                "head_dim": self.head_dim, "position": self.position.describe(prefix, ctx),
                "qk_norm_eps": self.qk_norm_eps, "window": int(self.window or 0), "scale": self.scale}
