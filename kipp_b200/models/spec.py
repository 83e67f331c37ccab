"""What a registered architecture builds from its configuration: the parts of
the model and the order in which its layers run."""
from __future__ import annotations

import dataclasses
from typing import Optional

from ..parts.base import Block, Norm, Part
from ..weights.spec import TensorSpec


@dataclasses.dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    ``layer``        index into ``ModelSpec.layers`` (a layer may be named twice);
    ``cache``        id of the cache (pages or state) this run uses; runs with the
                     same id share it;
    ``writes_cache`` False lets a run read the cache another run wrote
                     without adding its own keys and values.
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclasses.dataclass
class ModelSpec:
    config: object
    hidden_size: int
    vocab_size: int
    embedding: Part                  # parts.embedding.TokenEmbedding
    layers: list                     # list[(prefix, Block)]
    order: list                      # list[LayerRun]
    final_norm: tuple                # (prefix, Norm)
    head: tuple                      # (prefix, parts.embedding.OutputHead)
    embedding_prefix: str = "model.embed_tokens."
    max_positions: Optional[int] = None

    def tensor_specs(self) -> list[TensorSpec]:
        specs: list[TensorSpec] = []
        specs += self.embedding.tensor_specs(self.embedding_prefix)
        for prefix, block in self.layers:
            specs += block.tensor_specs(prefix)
        specs += self.final_norm[1].tensor_specs(self.final_norm[0])
        specs += self.head[1].tensor_specs(self.head[0])
        seen = set()
        for s in specs:
            if s.name in seen:
                raise ValueError(f"tensor {s.name} declared twice")
            seen.add(s.name)
        return specs

    @staticmethod
    def sequential_order(n_layers: int) -> list:
        return [LayerRun(layer=i, cache=i) for i in range(n_layers)]
