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
from .streams import ConnectedBlock, StreamConnection
from .latent_attention import LatentAttention
from .delta_rule import ChannelDeltaRule, HeadDeltaRule
from .norm import LayerNorm
from .routed_feed_forward import RoutedFeedForward
from .linear_recurrence import GatedLinearAttention, StateSpaceDuality
from .sandwich import SandwichBlock
from .position import YarnRotaryPositionEncoding
from .feed_forward import DenseFeedForward
from .differential_attention import DifferentialAttention
from .gated_residual import GatedResidualBlock

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "Part", "PartRegistryError", "PositionEncoding", "ScaledRows",
           "StepContext", "all_parts", "build_block", "build_part", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_part", "register_position_encoding", "registered", "unregister", "Linear", "RMSNorm", "NoPositionEncoding",
           "RotaryPositionEncoding", "llama3_inverse_frequencies", "GroupedQueryAttention", "SwiGLUFeedForward",
           "PreNormBlock", "OutputHead", "TokenEmbedding", "ConnectedBlock", "StreamConnection", "LatentAttention",
           "ChannelDeltaRule", "HeadDeltaRule", "LayerNorm", "RoutedFeedForward", "GatedLinearAttention",
           "StateSpaceDuality", "SandwichBlock", "YarnRotaryPositionEncoding", "DenseFeedForward",
           "DifferentialAttention", "GatedResidualBlock"]
