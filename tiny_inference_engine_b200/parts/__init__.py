"""The parts a model is assembled from, their registries, and the model built from a description."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheNeed, FeedForward, Mixer,
                   Norm, Part, PositionEncoding, StateNeed, build_part, register_part, to_compute)
from . import norm, position, attention, feed_forward, block  # noqa: F401  (register the built-in kinds)
from .attention import GQAttention
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feed_forward import SwiGLU
from .model import LayerCache, Model, expected_tensors
from .norm import RMSNorm
from .position import NoPositionEncoding, RotaryEncoding

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheNeed", "FeedForward",
           "Mixer", "Norm", "Part", "PositionEncoding", "StateNeed", "build_part", "register_part", "to_compute",
           "GQAttention", "PreNormBlock", "LMHead", "TokenEmbedding", "SwiGLU", "LayerCache", "Model",
           "expected_tensors", "RMSNorm", "NoPositionEncoding", "RotaryEncoding"]
