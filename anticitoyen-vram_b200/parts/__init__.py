"""Layer parts: mixers, feed-forwards, norms, position encodings, block arrangements."""

from .base import CacheView, FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, StepMetadata
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, default_schedule
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, build, register
from . import blocks, feed_forward, mixers, norms, position  # noqa: F401  (registers the built-in parts)

__all__ = ["BLOCKS", "CacheView", "FEED_FORWARDS", "FeedForward", "LayerSpec", "MIXERS", "Mixer", "ModelPlan",
           "NORMS", "Norm", "POSITION_ENCODINGS", "Part", "PartSpec", "PositionEncoding", "Runtime",
           "ScheduleEntry", "StepMetadata", "build", "default_schedule", "register"]
