"""Parts a decoder is assembled from; importing this package registers the
built-in kinds."""

from .base import (Block, CacheNeed, Embedding, FeedForward, Head, Mixer, Norm, ParamSpec, Part,
                   PartSpec, PositionEncoding, RotaryParams, WeightSource, build_part,
                   part_class, register_part, registered_parts)
from . import norms, positions, attention, feedforward, blocks, embedding  # noqa: F401  (registration)
