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
        """The checks are the host core's (csrc/host/qwen3.hpp): options the engine
        lacks are refused there, by name."""
        import json

        from .. import native as N
        N.text_result(N.lib().kipp_config_normalize, json.dumps(self.to_dict()).encode())
