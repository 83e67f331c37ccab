"""The parts a model is put together from, as Python sees them.

The parts themselves (their kernels' launch sequences, their weights on the
device) live in the host core (csrc/host/parts.hpp).  A Python part is one of
two things:

* a *description* of a part the library brings (``RMSNorm``, ``AttentionMixer``,
  ...): sizes and constants that become one JSON object of the model's plan;
* a part *defined in Python* (derive from ``Mixer``, ``FeedForward``, ``Norm`` or
  ``EmbeddingStage`` and write ``forward`` with torch calls on the tensors it is
  handed): the library calls it back inside the step.  Such a part declares its
  checkpoint tensors (``tensor_specs``), takes them in ``bind`` and may keep a
  fixed-size state per request (``state_spec``).  Its work is not captured in
  CUDA graphs unless it says ``graph_safe = True``.

Kinds of part and what a Python-defined one must provide:

``Norm``              ``forward(ctx, x_f32[T, size], out[rows, size], rows, n_rows)``
``PositionEncoding``  ``rotary_dim`` and ``frequencies()``: the rotation a mixer applies
                      to queries and keys at a token's absolute position (data, not a callback).
``Mixer``             ``state_spec()`` and ``forward(ctx, run, h, residual)``, which ADDS its
                      output to the float32 ``residual``.
``FeedForward``       ``forward(ctx, h, residual)``, which adds its output to ``residual``.
``EmbeddingStage``    ``forward(ctx, x)``: a stage at the bottom of the model that writes or
                      updates the residual stream ``x`` [T, hidden] (float32).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..weights.spec import TensorSpec


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


class PlanContext:
    """What describing a model collects: its hidden size (parts defined in
    Python are told it) and the Python-defined parts in the order of their index."""

    def __init__(self, hidden_size: int):
        self.hidden_size = hidden_size
        self.external: list = []          # (part, prefix)


class Part:
    """Base of every part.  ``kind`` names a part the library brings; a part with
    ``kind`` None is defined in Python and called back."""

    kind: Optional[str] = None
    role: Optional[str] = None            # of a Python-defined part: mixer, feed_forward, embedding, norm
    graph_safe = False

    # -- a library part -------------------------------------------------------
    def params(self, prefix: str, ctx: PlanContext) -> dict:
        """The JSON object of a library part (without its ``kind``)."""
        raise NotImplementedError

    # -- a Python-defined part ----------------------------------------------------
    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        if self.kind is not None:
            from ..models.spec import part_tensor_specs
            return part_tensor_specs(self, prefix)
        return []

    def bind(self, tensors, prefix: str, runtime) -> None:
        """Take declared tensors (CPU, storage dtype) and keep what forward needs."""

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def describe(self, prefix: str, ctx: PlanContext) -> dict:
        if self.kind is not None:
            return {"kind": self.kind, **self.params(prefix, ctx)}
        if self.role is None:
            raise TypeError(f"{type(self).__name__} is neither a library part nor a Mixer, FeedForward, Norm or "
                            "EmbeddingStage defined in Python")
        index = len(ctx.external)
        ctx.external.append((self, prefix))
        out = {"kind": "external", "role": self.role, "index": index, "hidden_size": ctx.hidden_size,
               "graph_safe": bool(self.graph_safe),
               "tensors": [{"name": s.name, "shape": list(s.shape), "init": s.init, "optional": s.optional,
                            "alias_of": s.alias_of, "ignore_if_present": s.ignore_if_present}
                           for s in self.tensor_specs(prefix)]}
        size = getattr(self, "size", None)
        if size is not None:
            out["size"] = int(size)
        ss = self.state_spec()
        if ss is not None:
            names = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.int32: "int32"}
            if ss.dtype not in names:
                raise TypeError("a state is float32, bfloat16 or int32")
            out["state"] = {"shape": list(ss.shape), "dtype": names[ss.dtype]}
        return out


class Norm(Part):
    role = "norm"

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor], n_rows: int) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    """A rotation given by frequencies: pair (i, i + rotary_dim/2) of a head turns
    by position * frequencies()[i].  Subclasses give ``rotary_dim``,
    ``frequencies()`` (float32 ``[rotary_dim // 2]``) and ``table_key()``:
    encodings with equal keys rotate alike and share a step's (cos, sin) table."""
    rotary_dim: int = 0

    def frequencies(self) -> Optional[torch.Tensor]:
        return None

    def table_key(self):
        return id(self)

    def describe(self, prefix: str, ctx: PlanContext) -> dict:
        f = self.frequencies()
        if f is None or self.rotary_dim == 0:
            return {"kind": "no_position"}
        return {"kind": "frequency_table", "inv_freq": [float(v) for v in f.float().tolist()],
                "key": repr(self.table_key())}


class Mixer(Part):
    role = "mixer"

    def cache_spec(self) -> Optional[PagedKVSpec]:
        return None

    def forward(self, ctx, run, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    role = "feed_forward"

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class EmbeddingStage(Part):
    role = "embedding"

    def forward(self, ctx, x: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
