"""Parts a model is put together from.  Importing the package registers the
built-in kinds; ``register_part`` / ``register_arrangement`` add others."""

from . import attention, block, embedding, mlp, norm  # noqa: F401  (register themselves)
from .base import (Arrangement, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding,
                   build_part, get_arrangement, register_arrangement, register_part)
from .spec import (FixedState, LayerSpec, ModelSpec, NoCache, PagedKV, PartSpec, RunEntry, WeightSpec)

__all__ = [
    "Arrangement", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
    "build_part", "get_arrangement", "register_arrangement", "register_part",
    "FixedState", "LayerSpec", "ModelSpec", "NoCache", "PagedKV", "PartSpec", "RunEntry", "WeightSpec",
]
