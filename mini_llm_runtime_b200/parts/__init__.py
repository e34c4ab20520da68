from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registers the parts)
from .base import (Block, Embedding, FeedForward, Head, KVCacheNeed, Mixer, Norm, Part,
                   PositionEncoding, StateNeed, TensorSpec, build_part, known_parts, part_factory,
                   register_part, unregister_part)

__all__ = [
    "Block", "Embedding", "FeedForward", "Head", "KVCacheNeed", "Mixer", "Norm", "Part",
    "PositionEncoding", "StateNeed", "TensorSpec", "build_part", "known_parts", "part_factory",
    "register_part", "unregister_part",
]
