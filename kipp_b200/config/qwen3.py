"""Configuration of the Qwen3 dense decoder, from its ``config.json`` keys.

The reference fixes 8 KV heads, head_dim 128, vocab 151,936 and eps 1e-6 in
code (src/kipp.h:19-21, src/kipp.c:29) and takes the other sizes from a
registry row (src/kipp_backend.h:19-34); the converter lists the matching
``config.json`` keys (tools/convert_to_gguf.py:471-485).  Here every one of
them is a field.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

from .base import ConfigError, ModelConfig

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclasses.dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    # head_dim may differ from hidden_size / num_attention_heads (the q width
    # is never conflated with the hidden width, src/kipp_backend.h:50-53).
    head_dim: Optional[int] = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    rope_scaling: Optional[dict] = None
    # Window options.  A layer with a window of w sees keys j with
    # pos - w < j <= pos.  The reference runs full attention only
    # (docs/ARCHITECTURE.md:48-57); the keys are honoured here because the
    # checkpoint format has them.
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[tuple] = None
    initializer_range: float = 0.02
    torch_dtype: str = "bfloat16"
    model_type: str = "qwen3"
    eos_token_id: Optional[int] = None

    json_aliases = {"torch_dtype": ("dtype",)}

    def __post_init__(self) -> None:
        if self.head_dim is None:
            if self.num_attention_heads <= 0 or self.hidden_size % self.num_attention_heads:
                raise ConfigError(
                    "head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)

    # -- derived sizes ----------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of layer ``layer`` in keys, or None for full attention."""
        if self.layer_types is not None:
            if self.layer_types[layer] == SLIDING_ATTENTION:
                return self.sliding_window
            return None
        if self.use_sliding_window and self.sliding_window is not None:
            first = self.max_window_layers if self.max_window_layers is not None else 0
            return self.sliding_window if layer >= first else None
        return None

    def validate(self) -> None:
        positive = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
                    "head_dim")
        for name in positive:
            if getattr(self, name) <= 0:
                raise ConfigError(f"config key {name!r} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotary pairs")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.attention_bias or self.mlp_bias:
            raise ConfigError("attention_bias / mlp_bias are not supported (Qwen3 dense has none)")
        if self.rope_scaling is not None:
            kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
            if kind not in (None, "default"):
                raise ConfigError(f"rope_scaling {kind!r} is not supported")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError("layer_types must have one entry per layer")
            for kind in self.layer_types:
                if kind not in (FULL_ATTENTION, SLIDING_ATTENTION):
                    raise ConfigError(f"unknown layer type {kind!r}")
            if SLIDING_ATTENTION in self.layer_types and not self.sliding_window:
                raise ConfigError("layer_types names sliding_attention but sliding_window is unset")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")
