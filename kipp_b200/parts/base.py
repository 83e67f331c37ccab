"""Interfaces of the parts a model is put together from.

A part is built from sizes and constants only; it never learns which model it
is in.  Its life has three stages:

1. construction from parameters (no device needed): ``tensor_specs(prefix)``
   already works, so checkpoints can be checked and random weights made;
2. ``bind(tensors, prefix, runtime)``: take the checkpoint tensors it declared,
   move them to the device in the form its kernels want;
3. ``forward(...)`` inside a step.

Kinds of part and what each must provide:

``Norm``              ``forward(ctx, x_f32[T, size]) -> h[T, size]`` in the compute dtype.
``PositionEncoding``  ``rotary_dim`` and ``inv_freq(device)``: the rotation a mixer applies
                      to queries and keys at a token's absolute position.
``Mixer``             ``cache_spec()`` (pages it needs, or None), ``state_spec()`` (fixed-size
                      per-request state, or None) and
                      ``forward(ctx, run, h, residual)``, which ADDS its output to the
                      float32 ``residual``.
``FeedForward``       ``forward(ctx, h, residual)``, which adds its output to ``residual``.
``Block``             the arrangement of the four in one layer:
                      ``forward(ctx, run, x)`` updates the residual stream ``x`` in place.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..weights.spec import TensorSpec


class Part:
    """Base of every part."""

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor], prefix: str, runtime) -> None:
        """Take declared tensors (CPU or device, storage dtype) and keep device copies."""

    def weight_bytes(self) -> int:
        """Bytes of weights one forward pass reads (for roofline accounting)."""
        return 0


@dataclasses.dataclass(frozen=True)
class PagedKVSpec:
    """Cache need of a mixer: keys and values of ``kv_heads`` heads of
    ``head_dim`` per token.  ``window`` None keeps every key; a window of w
    keeps keys j with pos - w < j <= pos.  Runs with equal specs share a group
    of the cache manager (own pool, own block tables, own retention)."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer: one tensor of ``shape`` and
    ``dtype`` per request, zeroed when a request is admitted."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    rotary_dim: int = 0

    def inv_freq(self, device) -> Optional[torch.Tensor]:
        """float32 ``[rotary_dim // 2]``: angle of pair i at position p is p * inv_freq[i]."""
        return None

    def table_key(self):
        """Encodings with equal keys rotate alike and share a step's (cos, sin) table."""
        return id(self)


class Mixer(Part):
    def cache_spec(self) -> Optional[PagedKVSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, ctx, run, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, ctx, run, x: torch.Tensor) -> None:
        raise NotImplementedError
