from . import attention, block, delta, embedding, feedforward, matrix_memory, norm, parallel, recurrent, retention, rope  # noqa: F401  (registers the parts)
from .block import Block, Branches
from .base import (FeedForward, KVNeed, LayerCache, Mixer, Part, Runtime, StateNeed, StepContext, StreamValue, build_part,
                   part_class, register_part)

__all__ = ["Block", "Branches", "StreamValue", "FeedForward", "KVNeed", "LayerCache", "Mixer", "Part", "Runtime", "StateNeed", "StepContext",
           "build_part", "part_class", "register_part"]
