"""Parts a decoder layer is assembled from (see :mod:`.base` for the interfaces)."""

from . import attention, block, embedding, moe, norm, position  # noqa: F401  (registers the kinds)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block,
                   CacheView, Embedding, FeedForward, Head, Mixer, Norm, Part, Position, Segment,
                   StepContext, StepPlan, StepShape, Workspace, register_block, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm,
                   register_position)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block",
    "CacheView", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "Position",
    "Segment", "StepContext", "StepPlan", "StepShape", "Workspace", "register_block", "register_embedding",
    "register_feed_forward", "register_head", "register_mixer", "register_norm",
    "register_position",
]
