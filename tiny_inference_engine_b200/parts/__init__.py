"""The parts a model is assembled from, their registries, and the model built from a description."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheNeed,
                   Embedding, FeedForward, Mixer, Norm, OutputHead, Part, PositionEncoding, StateNeed, build_part,
                   register_part, to_compute)
from . import norm, position, attention, feed_forward, block, embedding  # noqa: F401  (register the built-in kinds)
from .attention import GQAttention
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feed_forward import SwiGLU
from .model import LayerCache, Model, expected_tensors
from .norm import RMSNorm
from .position import NoPositionEncoding, RotaryEncoding

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheNeed",
           "Embedding", "FeedForward", "Mixer", "Norm", "OutputHead", "Part", "PositionEncoding", "StateNeed", "build_part", "register_part", "to_compute",
           "GQAttention", "PreNormBlock", "LMHead", "TokenEmbedding", "SwiGLU", "LayerCache", "Model",
           "expected_tensors", "RMSNorm", "NoPositionEncoding", "RotaryEncoding"]
