from . import (attention, block, chunk_attention, experts, latent_attention,  # noqa: F401
               mlp, norm, parallel, recurrent, rope, sink_attention, token_side,
               window_attention)  # (register the built-in kinds)
from .base import (Block, FeedForward, Mixer, Norm, PagedKVSpec, Part, PositionEncoding,
                   StateSpec, build_block, build_feed_forward, build_mixer, build_norm,
                   build_position_encoding, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position_encoding,
                   register_side_input)
from .context import CacheBinding, ResidualStream, StepContext, StepPrep, Workspace

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "PagedKVSpec", "Part", "PositionEncoding",
           "StateSpec", "build_block", "build_feed_forward", "build_mixer", "build_norm",
           "build_position_encoding", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding",
           "register_side_input", "CacheBinding",
           "ResidualStream", "StepContext", "StepPrep", "Workspace"]
