from .base import (Block, CacheSpec, FeedForward, FixedStateSpec, Mixer, Norm, PagedKVSpec, Part,
                   PositionEncoding, Rotation, WeightSlot)
from .linear import Linear
from .norm import RMSNorm
from .rotary import NoPositionEncoding, RotaryHalf, RotaryInterleaved
from .attention import GroupedQueryAttention
from .mlp import GatedMLP
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding

__all__ = ["Block", "CacheSpec", "FeedForward", "FixedStateSpec", "Mixer", "Norm", "PagedKVSpec", "Part",
           "PositionEncoding", "Rotation", "WeightSlot", "Linear", "RMSNorm", "NoPositionEncoding", "RotaryHalf", "RotaryInterleaved",
           "GroupedQueryAttention", "GatedMLP", "PreNormBlock", "LMHead", "TokenEmbedding"]
