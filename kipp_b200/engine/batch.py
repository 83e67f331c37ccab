"""One request's share of a step."""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass
class StepEntry:
    """One request's share of a step: its next ``tokens`` and the indices among
    them (``want``) whose logits are asked for."""
    request: object
    tokens: list
    want: list = dataclasses.field(default_factory=list)
