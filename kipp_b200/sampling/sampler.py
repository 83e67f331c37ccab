"""Turns the logits of a step into one token per wanted row, on the device.

The host keeps each request's generator state and draws the uniform number;
the kernels do everything that touches the vocabulary (penalties, maximum,
candidate cut, top-k, min-p, nucleus, the draw).  Both halves are the host
core's (Engine::sample, csrc/host/engine.hpp); this class is their face.
"""
from __future__ import annotations

from typing import Sequence

from .params import SamplingParams


class Sampler:
    def __init__(self, engine):
        self.engine = engine

    def sample(self, params: Sequence[SamplingParams], rng_states: list[int],
               recent: Sequence[Sequence[int]] | None = None) -> list[int]:
        """One token for each row of the engine's last logits (modified in place
        when a row has penalties or a bias).  ``rng_states[i]`` is advanced for rows
        with temperature > 0 only, as the reference leaves the generator
        untouched on the greedy path."""
        if len(rng_states) != len(params):
            raise ValueError("one SamplingParams and one generator state per row")
        return self.engine.sample(list(params), rng_states, recent)
