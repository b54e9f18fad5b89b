from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, SHIFTS, FeedForward,
                   GroupView, LayerCache, Mixer, Norm, OwedNorm, PagedKV, Part,
                   PositionEncoding, Registry, SlotState, StepContext, TensorSpec, flatten_needs)

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "SHIFTS", "FeedForward",
    "GroupView", "LayerCache", "Mixer", "Norm", "OwedNorm", "PagedKV", "Part",
    "PositionEncoding", "Registry", "SlotState", "StepContext", "TensorSpec", "flatten_needs",
]
