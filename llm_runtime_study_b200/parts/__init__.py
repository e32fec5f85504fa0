from . import attention, block, mlp, norm, rope  # registers the built-in kinds
from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, FixedState,
    Mixer, Norm, PagedKV, Part, PositionEncoding, Registry, ResidualStream, Runtime,
)
from .embedding import OutputHead, TokenEmbedding
from .linear import Projection

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "FeedForward",
    "FixedState", "Mixer", "Norm", "OutputHead", "PagedKV", "Part", "PositionEncoding", "Projection",
    "Registry", "ResidualStream", "Runtime", "TokenEmbedding",
]
