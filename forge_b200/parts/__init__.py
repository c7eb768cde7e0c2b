from .base import (CATEGORIES, KVCacheSpec, Part, Runtime, StateSpec, build_part, register_part, registered_parts,
                   unregister_part)
from . import attention, block, embedding, feedforward, norm, position  # noqa: F401  (register the built-in parts)
from .block import build_block
from .linear import Linear

__all__ = ["CATEGORIES", "KVCacheSpec", "StateSpec", "Part", "Runtime", "Linear", "build_part", "build_block",
           "register_part", "registered_parts", "unregister_part"]
