"""Parts a model is assembled from.  Importing this package registers the built-in ones."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, PASS_ENTRIES, POSITIONS, Block, PassEntry, CacheNeeds, FeedForward, LayerSpec,
                   Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, Registry, ResidualStream,
                   ScheduleEntry, StepContext, WeightSpec, build_block, build_part, default_schedule)
from .embedding import EMBEDDINGS, HEADS
from . import (attention, block, feedforward, latent_attention, linear_recurrence, norm, parallel, position, recurrent,  # noqa: F401
               repeat, talking_attention)

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "PASS_ENTRIES", "PassEntry", "POSITIONS", "EMBEDDINGS", "HEADS", "Block", "CacheNeeds",
    "FeedForward", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec", "PositionEncoding", "Registry",
    "ResidualStream", "ScheduleEntry", "StepContext", "WeightSpec", "build_block", "build_part",
    "default_schedule",
]
