"""The Qwen3 dense decoder as a list of parts chosen by its configuration.

Per layer: RMSNorm -> attention (q/k/v projections, per-head q/k RMSNorm,
rotary encoding, causal grouped-query attention, output projection) -> add ->
RMSNorm -> SwiGLU feed-forward -> add; then a final RMSNorm and the output
head, tied to the embedding or not (docs/ARCHITECTURE.md:77-92; tensor names
src/kipp.c:947-994; 2 + 11*L (+1) tensors, src/kipp.c:1108-1111).
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..parts import (AttentionMixer, OutputHead, PreNormBlock, RMSNorm, RotaryEncoding,
                     SwiGLUFeedForward, TokenEmbedding)
from .spec import ModelSpec


def build_qwen3(config: Qwen3Config) -> ModelSpec:
    c = config
    embedding = TokenEmbedding(c.vocab_size, c.hidden_size)
    layers = []
    for i in range(c.num_hidden_layers):
        mixer = AttentionMixer(
            c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            position=RotaryEncoding(c.head_dim, c.rope_theta),
            qk_norm_eps=c.rms_norm_eps, window=c.layer_window(i))
        block = PreNormBlock(RMSNorm(c.hidden_size, c.rms_norm_eps), mixer,
                             RMSNorm(c.hidden_size, c.rms_norm_eps),
                             SwiGLUFeedForward(c.hidden_size, c.intermediate_size))
        layers.append((f"model.layers.{i}.", block))
    head = OutputHead(c.vocab_size, c.hidden_size,
                      tied_to=embedding if c.tie_word_embeddings else None)
    return ModelSpec(config=c, hidden_size=c.hidden_size, vocab_size=c.vocab_size,
                     embedding=embedding, layers=layers,
                     order=ModelSpec.sequential_order(c.num_hidden_layers),
                     final_norm=("model.norm.", RMSNorm(c.hidden_size, c.rms_norm_eps)),
                     head=("lm_head.", head), max_positions=c.max_position_embeddings)


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3)
