from .base import FeedForward, Mixer, Norm, Part, PositionEncoding, TensorSpec
from .registry import build_block, build_part, register_part, registered_parts
from . import attention, block, embedding, norm, rotary, swiglu  # noqa: F401  (registers the built-in parts)

__all__ = ["FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "TensorSpec", "build_part", "register_part",
           "registered_parts", "build_block"]
