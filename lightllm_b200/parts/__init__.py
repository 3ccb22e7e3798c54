"""Parts that layers are put together from.  Importing this package registers the built-in ones."""
from .base import CacheView, FeedForward, Mixer, Norm, Part, PositionEncoding
from .attention import AttentionMixer
from .block import Block, build_part
from .conv_attention import ConvAttentionMixer
from .delta import ChannelDeltaMixer
from .differential_attention import DifferentialAttentionMixer
from .sink_attention import KeyValuedAttentionMixer
from .moe import RoutedExperts
from .stream import StreamReinjection, StreamStepVector
from .input_conv import CausalInputConv
from .mixed_heads_attention import MixedHeadsAttention
from .matrix_memory import MatrixMemoryMixer
from .joined_mixers import JoinedMixers
from .embedding import LMHead, TokenEmbedding
from .gated_attention import GatedAttentionMixer, LatentAttentionMixer
from .mlp import GatedMLP
from .norm import LayerNorm, RMSNorm
from .retention import RetentionMixer
from .rotary import NoPositionEncoding, RotaryEmbedding

__all__ = ["CacheView", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "AttentionMixer", "Block",
           "build_part", "LMHead", "TokenEmbedding", "GatedMLP", "RMSNorm", "LayerNorm", "GatedAttentionMixer",
           "LatentAttentionMixer", "RetentionMixer", "NoPositionEncoding", "RotaryEmbedding", "ConvAttentionMixer",
           "ChannelDeltaMixer", "RoutedExperts", "StreamReinjection", "StreamStepVector", "CausalInputConv",
           "MixedHeadsAttention", "MatrixMemoryMixer", "JoinedMixers", "DifferentialAttentionMixer",
           "KeyValuedAttentionMixer"]
