"""What a registered architecture builds from its configuration: the parts of
the model and the order in which its layers run.  ``to_plan`` turns it into the
JSON plan the host core builds its parts from (csrc/host/model.hpp)."""
from __future__ import annotations

import dataclasses
import json
from typing import Optional

from .. import native as N
from ..parts.base import Part, PlanContext
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


def _specs_from_json(text: str) -> list[TensorSpec]:
    return [TensorSpec(s["name"], tuple(s["shape"]), s.get("init", "normal"), bool(s.get("optional", False)),
                       s.get("alias_of"), bool(s.get("ignore_if_present", False)))
            for s in json.loads(text)]


def part_tensor_specs(part: Part, prefix: str) -> list[TensorSpec]:
    """The checkpoint tensors one part declares under a name prefix."""
    described = part.describe(prefix, PlanContext(int(getattr(part, "hidden_size", 0) or 0)))
    return _specs_from_json(N.text_result(N.lib().kipp_part_tensor_specs, json.dumps(described).encode(),
                                          prefix.encode()))


@dataclasses.dataclass
class ModelSpec:
    """``embedding`` is one stage or a list of (prefix, stage): the first writes
    the residual stream from the token ids, later ones may add to it."""
    config: object
    hidden_size: int
    vocab_size: int
    embedding: object                # a part, or list[(prefix, part)]
    layers: list                     # list[(prefix, Block)]
    order: list                      # list[LayerRun]
    final_norm: tuple                # (prefix, Norm)
    head: tuple                      # (prefix, parts.embedding.OutputHead)
    embedding_prefix: str = ""       # prefix of a single embedding stage
    max_positions: Optional[int] = None
    plan: Optional[dict] = None      # a plan made by the library's own builder stands for the parts

    def embedding_stages(self) -> list:
        if isinstance(self.embedding, (list, tuple)):
            return list(self.embedding)
        return [(self.embedding_prefix, self.embedding)]

    def to_plan(self) -> tuple[dict, list]:
        """(plan, the Python-defined parts with their prefixes in the order of their index)."""
        if self.plan is not None:
            return self.plan, []
        ctx = PlanContext(self.hidden_size)
        cfg = self.config.to_dict() if hasattr(self.config, "to_dict") else None
        plan = {
            "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
            "max_positions": self.max_positions, "config": cfg,
            "embedding": [{"prefix": p, "part": part.describe(p, ctx)} for p, part in self.embedding_stages()],
            "layers": [{"prefix": p, "part": block.describe(p, ctx)} for p, block in self.layers],
            "order": [{"layer": r.layer, "cache": r.cache, "writes_cache": r.writes_cache} for r in self.order],
            "final_norm": {"prefix": self.final_norm[0], "part": self.final_norm[1].describe(self.final_norm[0], ctx)},
            "head": {"prefix": self.head[0], "part": self.head[1].describe(self.head[0], ctx)},
        }
        return plan, ctx.external

    def tensor_specs(self) -> list[TensorSpec]:
        plan, _ = self.to_plan()
        return _specs_from_json(N.text_result(N.lib().kipp_plan_tensor_specs, json.dumps(plan).encode()))

    @staticmethod
    def sequential_order(n_layers: int) -> list:
        return [LayerRun(layer=i, cache=i) for i in range(n_layers)]

    @classmethod
    def from_library(cls, config) -> "ModelSpec":
        """The plan the library's own builder makes for ``config`` (an
        architecture registered in the host core)."""
        plan = json.loads(N.text_result(N.lib().kipp_plan_from_config, json.dumps(config.to_dict()).encode()))
        return cls(config=config, hidden_size=plan["hidden_size"], vocab_size=plan["vocab_size"],
                   embedding=None, layers=[], order=[LayerRun(o["layer"], o["cache"], o["writes_cache"])
                                                     for o in plan["order"]],
                   final_norm=(plan["final_norm"]["prefix"], None), head=(plan["head"]["prefix"], None),
                   max_positions=plan.get("max_positions"), plan=plan)
