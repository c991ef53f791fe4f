"""Layer parts: mixers, feed-forwards, norms, position encodings and block
arrangements, each chosen per layer by the layout's specs."""
from .base import (CacheNeed, KVNeed, LayerCache, ResidualStream, Runtime, StateNeed,
                   StepContext)
from .registry import build_part, known_parts, part_class, register_part, unregister_part

__all__ = ["CacheNeed", "KVNeed", "LayerCache", "ResidualStream", "Runtime", "StateNeed",
           "StepContext", "build_part", "known_parts", "part_class", "register_part",
           "unregister_part"]
