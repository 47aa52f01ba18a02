from . import attention, block, mlp, norm, rope  # noqa: F401  (register the built-in kinds)
from .base import (Block, FeedForward, Mixer, Norm, PagedKVSpec, Part, PositionEncoding,
                   StateSpec, build_block, build_feed_forward, build_mixer, build_norm,
                   build_position_encoding, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position_encoding)
from .context import CacheBinding, ResidualStream, StepContext, StepPrep, Workspace

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "PagedKVSpec", "Part", "PositionEncoding",
           "StateSpec", "build_block", "build_feed_forward", "build_mixer", "build_norm",
           "build_position_encoding", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding", "CacheBinding",
           "ResidualStream", "StepContext", "StepPrep", "Workspace"]
