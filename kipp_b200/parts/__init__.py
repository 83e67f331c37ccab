from .attention import AttentionMixer
from .base import (Block, EmbeddingStage, FeedForward, Mixer, Norm, PagedKVSpec, Part, PlanContext,
                   PositionEncoding, StateSpec)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .mlp import SwiGLUFeedForward
from .norm import RMSNorm
from .rope import NoPositionEncoding, RotaryEncoding

__all__ = ["AttentionMixer", "Block", "EmbeddingStage", "FeedForward", "Mixer", "Norm", "PagedKVSpec", "Part",
           "PlanContext", "PositionEncoding", "StateSpec", "PreNormBlock", "OutputHead", "TokenEmbedding",
           "SwiGLUFeedForward", "RMSNorm", "NoPositionEncoding", "RotaryEncoding"]
