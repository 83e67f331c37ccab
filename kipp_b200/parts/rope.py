"""Rotary position encoding with half-split pairs (src/kipp.c:2368-2382):
pair (i, i + rot/2) of a head is rotated by position * theta^(-2i/rot)."""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
    """``rotary_dim`` leading dims of each head are rotated (all of them by
    default); ``theta`` is the frequency base."""
    kind = "rotary"

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")

    def frequencies(self) -> torch.Tensor:
        """float32 theta^(-2i/rot) for i < rot/2, as the reference's
        powf(theta, -(2.0f * i) / rot): a float32 exponent, the power rounded
        to float32 once (the library computes the same values)."""
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float32)
        exponent = (-(2.0 * i) / float(self.rotary_dim)).double()
        theta = torch.tensor(self.theta, dtype=torch.float32).double()
        return torch.pow(theta, exponent).float()

    def table_key(self):
        return ("rotary", self.theta, self.rotary_dim)

    def describe(self, prefix, ctx) -> dict:
        if self.rotary_dim == 0:
            return {"kind": "no_position"}
        return {"kind": "rotary", "head_dim": self.head_dim, "theta": self.theta, "rotary_dim": self.rotary_dim}


class NoPositionEncoding(PositionEncoding):
    rotary_dim = 0

    def inv_freq(self, device=None):
        return None
