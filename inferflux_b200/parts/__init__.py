"""The parts layers are made of.  Importing the package registers the built-in kinds."""
from .base import (Block, FeedForward, KVCacheSpec, Mixer, Norm, Part, PositionEncoding, RotaryTable,
                   StateSpec, WeightBuffers, build_part, register_part, registered_parts)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)

__all__ = ["Block", "FeedForward", "KVCacheSpec", "Mixer", "Norm", "Part", "PositionEncoding",
           "RotaryTable", "StateSpec", "WeightBuffers", "build_part", "register_part", "registered_parts"]
