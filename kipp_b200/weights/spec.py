"""Declaration of one checkpoint tensor a part needs."""
from __future__ import annotations

import dataclasses

# How a tensor is initialised in random-weights mode.
INIT_NORMAL = "normal"            # N(0, sigma)
INIT_NEAR_ONE = "near_one"        # 1 + U(-a, a): norm scales
INIT_INT = "int"                  # integer table


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """``name`` is the checkpoint's tensor name, ``shape`` its exact shape.

    ``optional`` tensors may be absent (a tied output head); ``alias_of`` names
    the tensor that stands in when this one is absent.
    """
    name: str
    shape: tuple[int, ...]
    init: str = INIT_NORMAL
    optional: bool = False
    alias_of: str | None = None
    ignore_if_present: bool = False
