"""Parts that layers are put together from.  Importing this package registers the built-in kinds."""
from .base import (TensorSpec, KVCacheSpec, StateCacheSpec, CompositeCacheSpec, RunContext, Part, Norm,
                   PositionEncoding, Mixer, FeedForward, TokenInput, PartSpec)
from .registry import register_part, build_part
from . import norm, rotary, attention, latent_attention, feedforward, recurrent, parallel, token_input  # noqa: F401  (register themselves)
from .block import Arrangement, LayerSpec, PreNormBlock, build_layer
from . import streams  # noqa: F401
from .model import LayerCall, ModelSpec, Model

__all__ = ["TensorSpec", "KVCacheSpec", "StateCacheSpec", "CompositeCacheSpec", "TokenInput", "RunContext", "Part", "Norm", "PositionEncoding",
           "Mixer", "FeedForward", "PartSpec", "register_part", "build_part", "LayerSpec", "Arrangement", "PreNormBlock",
           "build_layer", "LayerCall", "ModelSpec", "Model"]
