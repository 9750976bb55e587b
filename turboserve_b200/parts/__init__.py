"""Parts a model is put together from; importing the package registers the built-in kinds."""

from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, FeedForward, LogitHead, Mixer, Norm, PagedKVNeed,
    ParamSpec, Part, PositionEncoding, StateNeed, TokenEmbedding, register_block, register_embedding, register_feed_forward,
    register_head, register_mixer, register_norm, register_position,
)
from . import attention, block, mlp, norm, rope, vocabulary  # noqa: F401,E402  (registration)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "FeedForward", "LogitHead", "Mixer",
    "Norm", "PagedKVNeed", "ParamSpec", "Part", "PositionEncoding", "StateNeed", "TokenEmbedding", "register_block",
    "register_embedding", "register_feed_forward", "register_head", "register_mixer", "register_norm", "register_position",
]
