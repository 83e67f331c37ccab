"""Sampling options of one request, with the reference's names and defaults
(kipp_sample_params, src/kipp.h:278-291; CLI flags src/kipp_cli.c:571-610)."""
from __future__ import annotations

import dataclasses

RECENT_WINDOW = 64          # tokens the penalties look back over (src/kipp_server.c:869-887)
MASK64 = (1 << 64) - 1


@dataclasses.dataclass
class SamplingParams:
    temperature: float = 0.0          # 0 = greedy argmax
    top_p: float = 1.0                # nucleus mass, 0 < top_p <= 1
    top_k: int = 0                    # keep the k highest logits, 0 = off
    min_p: float = 0.0                # min probability relative to the top, 0 = off
    seed: int = 1                     # nonzero seed of the request's generator
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: dict = dataclasses.field(default_factory=dict)   # token id -> added logit

    def validate(self) -> None:
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be greater than 0 and at most 1")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be between 0 and 1")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if self.temperature > 0.0 and (self.seed & MASK64) == 0:
            raise ValueError("sampling requires a nonzero seed")

    @property
    def has_penalties(self) -> bool:
        return (self.frequency_penalty != 0.0 or self.presence_penalty != 0.0 or
                (self.repetition_penalty != 0.0 and self.repetition_penalty != 1.0))


def xorshift64_star(state: int) -> tuple[int, int]:
    """One step of the reference's generator (src/kipp.c:3322-3329):
    returns (new state, output)."""
    x = state & MASK64
    x ^= x >> 12
    x ^= (x << 25) & MASK64
    x ^= x >> 27
    return x, (x * 2685821657736338717) & MASK64


def next_uniform(state: int) -> tuple[int, float]:
    """(new state, uniform in [0, 1) with 53 bits) (src/kipp.c:3331-3333)."""
    state, r = xorshift64_star(state)
    return state, (r >> 11) / 9007199254740992.0


def to_native(params, recent=None):
    """The library's array of sampling options for rows with these ``SamplingParams``
    (and the tokens each row's penalties look back over); returns (array, what
    must stay alive while it is used)."""
    import ctypes

    from .. import native as N
    rows = len(params)
    arr = (N.SampleParams * max(rows, 1))()
    keep = []
    for i, p in enumerate(params):
        p.validate()
        a = arr[i]
        a.temperature, a.top_p, a.top_k, a.min_p = p.temperature, p.top_p, p.top_k, p.min_p
        a.frequency_penalty, a.presence_penalty = p.frequency_penalty, p.presence_penalty
        a.repetition_penalty = p.repetition_penalty
        r = list(recent[i])[-RECENT_WINDOW:] if recent is not None and p.has_penalties else []
        if r:
            buf = (ctypes.c_int32 * len(r))(*[int(t) for t in r])
            keep.append(buf)
            a.recent_tokens, a.recent_count = buf, len(r)
        if p.logit_bias:
            toks = (ctypes.c_int32 * len(p.logit_bias))(*[int(t) for t in p.logit_bias])
            vals = (ctypes.c_float * len(p.logit_bias))(*[float(v) for v in p.logit_bias.values()])
            keep += [toks, vals]
            a.logit_bias_tokens, a.logit_bias_values, a.logit_bias_count = toks, vals, len(p.logit_bias)
    return arr, keep
