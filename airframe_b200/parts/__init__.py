"""Parts of a layer and their registry; importing the package registers the
built-in kinds."""
from .base import (CATEGORIES, Block, BuildContext, FeedForward, KVNeed, Mixer, Norm, Part,
                   PositionEncoding, StateNeed, build_part, known_parts, register_part,
                   unregister_part)
from . import attention, block, ends, mlp, norm, rope  # noqa: F401  (registration)
from .linear import linear

__all__ = ["CATEGORIES", "Block", "BuildContext", "FeedForward", "KVNeed", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateNeed", "build_part", "known_parts", "register_part",
           "unregister_part", "linear"]
