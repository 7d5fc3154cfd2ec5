from . import attention, block, ends, rmsnorm, rope, swiglu  # noqa: F401  (registers the built-in kinds)
from .base import (CATEGORIES, CacheRequest, Embedding, FeedForward, Head, Layer, Mixer, Norm, Part, PositionEncoding, StateRequest,
                   TensorDecl, build_part, register_part, registered_parts)
from .model import DecoderModel
from .runtime import ResidualStream, Runtime

__all__ = ["CATEGORIES", "CacheRequest", "Embedding", "FeedForward", "Head", "Layer", "Mixer", "Norm", "Part", "PositionEncoding",
           "StateRequest", "TensorDecl", "build_part", "register_part", "registered_parts", "DecoderModel",
           "ResidualStream", "Runtime"]
