"""Arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from ..weights.spec import TensorSpec
from .base import Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x)) — the un-normed x is the
    residual stream (src/kipp.c:2948, 2994)."""

    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, ffn: FeedForward,
                 names: tuple[str, str, str, str] = ("input_layernorm.", "self_attn.",
                                                     "post_attention_layernorm.", "mlp.")):
        self.input_norm, self.mixer, self.post_norm, self.ffn = input_norm, mixer, post_norm, ffn
        self.names = names

    def _parts(self, prefix: str):
        return zip((self.input_norm, self.mixer, self.post_norm, self.ffn),
                   (prefix + n for n in self.names))

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [s for part, p in self._parts(prefix) for s in part.tensor_specs(p)]

    def bind(self, tensors, prefix, runtime) -> None:
        for part, p in self._parts(prefix):
            part.bind(tensors, p, runtime)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part, _ in self._parts(""))

    def forward(self, ctx, run, x) -> None:
        h = self.input_norm.forward(ctx, x)
        self.mixer.forward(ctx, run, h, x)
        h = self.post_norm.forward(ctx, x)
        self.ffn.forward(ctx, h, x)
