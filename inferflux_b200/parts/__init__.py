"""The parts layers are made of.  Importing the package registers the built-in kinds."""
from .base import (Block, FeedForward, KVCacheSpec, Mixer, Norm, NormedDelta, Part, PositionEncoding, RotaryTable,
                   StateSpec, StreamMerge, TimeConv, TokenInput, VectorScaledDelta, WeightBuffers, build_part, register_part, registered_parts,
                   settle_pending)
from . import (attention, block, conv, delta_rule, embedding, latent_attention, linear_scan, mlp, moe, norm, pair, rope,
               token_input, wkv)  # noqa: F401  (registration)

__all__ = ["Block", "FeedForward", "KVCacheSpec", "Mixer", "Norm", "NormedDelta", "Part", "PositionEncoding",
           "RotaryTable", "StateSpec", "VectorScaledDelta", "StreamMerge", "TimeConv", "TokenInput", "WeightBuffers", "build_part", "register_part",
           "registered_parts", "settle_pending"]
