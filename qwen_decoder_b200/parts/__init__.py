from .base import (Block, FeedForward, Mixer, Norm, PagedCacheView, Part, PositionEncoding, ResidualStream,
                   StateCacheView)
from .linear import Linear
from .model import DecoderModel, build_model
from .attention import GQAttention
from .mlp import SwiGLU
from .norm import RMSNorm
from .rotary import Rotary
from .block import PreNormBlock

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "PagedCacheView", "Part", "PositionEncoding",
           "ResidualStream", "StateCacheView", "Linear", "DecoderModel", "build_model", "GQAttention",
           "SwiGLU", "RMSNorm", "Rotary", "PreNormBlock"]
