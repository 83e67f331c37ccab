"""Token embedding and output head.

x_t = float(E[id_t, :]) with no scale (src/kipp.c:2940-2942); logits = W_lm n
for the wanted rows only, W_lm being the embedding when tied
(src/kipp.c:951-956, 3013-3018).  The parts themselves: csrc/host/parts.hpp."""
from __future__ import annotations

from typing import Optional

from .base import EmbeddingStage, Part


class TokenEmbedding(EmbeddingStage):
    kind = "token_embedding"

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size

    def params(self, prefix, ctx) -> dict:
        return {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}


class OutputHead(Part):
    """``tied_to`` names the checkpoint tensor (an embedding matrix) that stands
    in when the checkpoint has no head of its own."""
    kind = "output_head"

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to

    def params(self, prefix, ctx) -> dict:
        return {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied_to": self.tied_to}
