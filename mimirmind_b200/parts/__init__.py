"""The parts layers are made of.  Importing this package registers the built-in kinds."""
from . import attention, block, connections, differential_attention, embedding, latent_attention, linear_state, mingru, mlp, moe, norm, parallel_mixers, rope, sink_attention, talking_attention  # noqa: F401
from .base import (Block, CacheArray, FeedForward, KVCacheSpec, LayerCache, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StateSpec, StepContext, WeightView)

__all__ = ["Block", "CacheArray", "FeedForward", "KVCacheSpec", "LayerCache", "Mixer", "Norm", "Part", "PositionEncoding",
           "Runtime", "StateSpec", "StepContext", "WeightView"]
