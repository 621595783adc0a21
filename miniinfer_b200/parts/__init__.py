from .base import (Block, Embedding, FeedForward, Head, HostStep, Mixer, Norm, ParamSpec, Part, Piece, PositionEncoding,
                   StepWork, whole)
from .block import ParallelBlock, PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feedforward import RoutedExpertsFeedForward, SwiGLUFeedForward
from .gated_attention import GatedAttentionMixer
from .mixer import AttentionMixer
from .norm import LayerNorm, RMSNorm
from .position import RotaryEncoding
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, make, register_block,
                       register_feed_forward, register_mixer, register_norm, register_position_encoding)

register_mixer("attention")(AttentionMixer)
register_mixer("gated_attention")(GatedAttentionMixer)
register_feed_forward("swiglu")(SwiGLUFeedForward)
register_feed_forward("routed_experts")(RoutedExpertsFeedForward)
register_norm("rmsnorm")(RMSNorm)
register_norm("layernorm")(LayerNorm)
register_position_encoding("rotary")(RotaryEncoding)
register_block("pre_norm")(PreNormBlock)
register_block("parallel")(ParallelBlock)
