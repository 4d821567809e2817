from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, PartRegistry
from .base import Block, EntryCache, FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime
from . import attention, block, mlp, norm, rope  # noqa: F401  (registers the built-in parts)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "PartRegistry", "Block", "EntryCache",
           "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime"]
