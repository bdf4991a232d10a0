"""Parts that layers are put together from.  Importing this package registers the built-in ones."""
from .base import CacheView, FeedForward, Mixer, Norm, Part, PositionEncoding
from .attention import AttentionMixer
from .block import Block, build_part
from .embedding import LMHead, TokenEmbedding
from .mlp import GatedMLP
from .norm import RMSNorm
from .rotary import NoPositionEncoding, RotaryEmbedding

__all__ = ["CacheView", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "AttentionMixer", "Block",
           "build_part", "LMHead", "TokenEmbedding", "GatedMLP", "RMSNorm", "NoPositionEncoding", "RotaryEmbedding"]
