from .base import (Block, Embedding, FeedForward, Head, HostStep, Mixer, Norm, ParamSpec, Part, Piece, PositionEncoding,
                   StepWork, whole)
from .block import ParallelBlock, PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feedforward import RoutedExpertsFeedForward, SwiGLUFeedForward
from .gated_attention import GatedAttentionMixer
from .latent_attention import LatentAttentionMixer
from .mixer import AttentionMixer
from .norm import LayerNorm, RMSNorm
from .position import RotaryEncoding, ScaledRotaryEncoding
from .recurrent import GatedDeltaMixer, SelectiveScanMixer
from .side_by_side import SideBySideMixer
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, make, register_block,
                       register_feed_forward, register_mixer, register_norm, register_position_encoding)

register_mixer("attention")(AttentionMixer)
register_mixer("gated_attention")(GatedAttentionMixer)
register_mixer("latent_attention")(LatentAttentionMixer)
register_mixer("selective_scan")(SelectiveScanMixer)
register_mixer("gated_delta")(GatedDeltaMixer)
register_mixer("side_by_side")(SideBySideMixer)
register_feed_forward("swiglu")(SwiGLUFeedForward)
register_feed_forward("routed_experts")(RoutedExpertsFeedForward)
register_norm("rmsnorm")(RMSNorm)
register_norm("layernorm")(LayerNorm)
register_position_encoding("rotary")(RotaryEncoding)
register_position_encoding("scaled_rotary")(ScaledRotaryEncoding)
register_block("pre_norm")(PreNormBlock)
register_block("parallel")(ParallelBlock)
