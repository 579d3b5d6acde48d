from .base import (CacheSpec, CacheView, Part, Runtime, StateSpec, StateView, TensorDecl, WeightSource,
                   build_part, register_part, registered_parts)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .block import build_block
from .linear import Linear

__all__ = ["CacheSpec", "CacheView", "Part", "Runtime", "StateSpec", "StateView", "TensorDecl", "WeightSource",
           "build_part", "build_block", "register_part", "registered_parts", "Linear"]
