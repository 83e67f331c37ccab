from .attention import AttentionMixer
from .base import (Block, FeedForward, Mixer, Norm, PagedKVSpec, Part, PositionEncoding, StateSpec)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .mlp import SwiGLUFeedForward
from .norm import RMSNorm
from .rope import NoPositionEncoding, RotaryEncoding

__all__ = ["AttentionMixer", "Block", "FeedForward", "Mixer", "Norm", "PagedKVSpec", "Part",
           "PositionEncoding", "StateSpec", "PreNormBlock", "OutputHead", "TokenEmbedding",
           "SwiGLUFeedForward", "RMSNorm", "NoPositionEncoding", "RotaryEncoding"]
