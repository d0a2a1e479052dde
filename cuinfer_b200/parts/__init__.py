"""Parts a layer is made of, their registries, and the model built from a spec."""
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding, ResidualStream
from .context import GroupView, PagedKV, StepContext
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from .spec import LayerSpec, ModelSpec, PagedCacheNeed, PartSpec, StateNeed, TensorSpec

# importing the built-in parts registers them
from . import attention, block, feed_forward, norm, position  # noqa: E402,F401
from .model import DecoderModel, build_layer  # noqa: E402

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "ResidualStream",
    "GroupView", "PagedKV", "StepContext",
    "LayerSpec", "ModelSpec", "PagedCacheNeed", "PartSpec", "StateNeed", "TensorSpec",
    "DecoderModel", "build_layer",
]
