"""Parts a decoder is composed of, their specifications and registries."""
from . import specs
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Part, Registry, Runtime
from . import norm, position, attention, feedforward, block, embedding  # register the built-in kinds

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Part", "Registry", "Runtime", "specs"]
