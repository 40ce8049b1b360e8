"""Parts a layer is put together from, and their registries."""
from .base import (Block, FeedForward, Mixer, Norm, Part, PartRegistryError, PositionEncoding, ScaledRows, StepContext,
                   all_parts, build_block, build_part, register_block, register_feed_forward, register_mixer,
                   register_norm, register_part, register_position_encoding, registered, unregister)
from .linear import Linear
from .norm import RMSNorm
from .position import NoPositionEncoding, RotaryPositionEncoding, llama3_inverse_frequencies
from .attention import GroupedQueryAttention
from .feed_forward import SwiGLUFeedForward
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "Part", "PartRegistryError", "PositionEncoding", "ScaledRows",
           "StepContext", "all_parts", "build_block", "build_part", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_part", "register_position_encoding", "registered", "unregister", "Linear", "RMSNorm", "NoPositionEncoding",
           "RotaryPositionEncoding", "llama3_inverse_frequencies", "GroupedQueryAttention", "SwiGLUFeedForward",
           "PreNormBlock", "OutputHead", "TokenEmbedding"]
