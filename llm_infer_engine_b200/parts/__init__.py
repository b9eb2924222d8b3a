from .base import (AttentionOptions, Block, DeferredBranchAdd, DeferredNorm, FeedForward, Mixer, Norm, ParamSpec, Part, Pointwise, PositionEncoding, Runtime, ScaledDelta,
                   build_part, call_branch, lookup, register_block, register_feed_forward, register_mixer,
                   register_norm, register_pointwise, register_position_encoding, undefer)
from . import attention, block, embedding_stage, gated_attention, latent_attention, mlp, moe, norm, recurrent, rope, scaled  # noqa: F401  (register the built-in parts)
from .linear import Linear

__all__ = ["AttentionOptions", "Block", "DeferredBranchAdd", "DeferredNorm", "undefer", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "Pointwise",
           "PositionEncoding", "Runtime", "ScaledDelta", "build_part", "call_branch", "lookup", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_pointwise", "register_position_encoding", "Linear"]
