from .base import (Block, CacheTensor, FeedForward, KVNeed, Mixer, Norm, PagedNeed, Part, PositionEncoding, StateNeed,
                   build_block, build_part, register_part)
from .norm import RMSNorm
from .rope import NoPositionEncoding, RotaryEncoding
from .attention import GQAttention
from .mlp import SwiGLU
from .block import PreNormBlock

__all__ = ["Block", "CacheTensor", "FeedForward", "KVNeed", "Mixer", "Norm", "PagedNeed", "Part", "PositionEncoding",
           "StateNeed",
           "build_block", "build_part", "register_part", "RMSNorm", "NoPositionEncoding", "RotaryEncoding",
           "GQAttention", "SwiGLU", "PreNormBlock"]
