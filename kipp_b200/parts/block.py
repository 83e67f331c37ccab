"""Arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x)): the un-normed x is the
    residual stream (src/kipp.c:2948, 2994).  The part itself:
    csrc/host/parts.hpp."""
    kind = "pre_norm_block"

    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, ffn: FeedForward,
                 names: tuple[str, str, str, str] = ("input_layernorm.", "self_attn.",
                                                     "post_attention_layernorm.", "mlp.")):
        self.input_norm, self.mixer, self.post_norm, self.ffn = input_norm, mixer, post_norm, ffn
        self.names = tuple(names)

    def params(self, prefix, ctx) -> dict:
        parts = (self.input_norm, self.mixer, self.post_norm, self.ffn)
        described = [p.describe(prefix + n, ctx) for p, n in zip(parts, self.names)]
        return {"names": list(self.names), "input_norm": described[0], "mixer": described[1],
                "post_norm": described[2], "ffn": described[3]}
