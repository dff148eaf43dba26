from .base import (AttentionOptions, Block, DeferredNorm, FeedForward, Mixer, Norm, ParamSpec, Part, Pointwise, PositionEncoding, Runtime,
                   build_part, call_branch, lookup, register_block, register_feed_forward, register_mixer,
                   register_norm, register_pointwise, register_position_encoding, undefer)
from . import attention, block, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .linear import Linear

__all__ = ["AttentionOptions", "Block", "DeferredNorm", "undefer", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "Pointwise",
           "PositionEncoding", "Runtime", "build_part", "call_branch", "lookup", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_pointwise", "register_position_encoding", "Linear"]
