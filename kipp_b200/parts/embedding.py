"""Token embedding and output head.

x_t = float(E[id_t, :]) with no scale (src/kipp.c:2940-2942); logits = W_lm n
for the wanted rows only, W_lm being the embedding when tied
(src/kipp.c:951-956, 3013-3018)."""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.spec import TensorSpec
from .base import Part


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + "weight", (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, prefix, runtime) -> None:
        self.weight = tensors[prefix + "weight"].to(runtime.device).to(runtime.dtype).contiguous()

    def forward(self, ctx) -> torch.Tensor:
        T = ctx.meta.tokens
        x = ctx.workspace.buffer("residual", (T, self.hidden_size), torch.float32)
        ctx.ops.embed_gather(x, self.weight, ctx.meta.token_ids, ctx.status)
        return x


class OutputHead(Part):
    """``tied_to`` is the TokenEmbedding whose matrix stands in when the
    checkpoint has no head of its own."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[TokenEmbedding] = None,
                 tied_name: str = "model.embed_tokens.weight"):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to
        self.tied_name = tied_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        if self.tied_to is not None:
            return [TensorSpec(prefix + "weight", (self.vocab_size, self.hidden_size), optional=True,
                               alias_of=self.tied_name, ignore_if_present=True)]
        return [TensorSpec(prefix + "weight", (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, prefix, runtime) -> None:
        if self.tied_to is not None:
            self.weight = self.tied_to.weight
        else:
            self.weight = tensors[prefix + "weight"].to(runtime.device).to(runtime.dtype).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx, h: torch.Tensor, n_rows: int) -> torch.Tensor:
        logits = ctx.workspace.buffer("logits", (n_rows, self.vocab_size), torch.float32)
        ctx.ops.gemm(logits, h, self.weight, "store", m=n_rows)
        return logits
