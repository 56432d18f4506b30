"""The parts layers are put together from: norm, position encoding, mixer, feed-forward, block,
embedding and head.  Importing this package registers the built-in kinds."""
from .base import CacheNeed, Part, Runtime, StepContext
from .linear import Linear
from .norm import DynamicTanh, DynamicTanhSpec, RMSNorm, RMSNormSpec
from .position import Llama3Scaling, NoPosition, NoPositionSpec, Rotary, RotarySpec, rotary_inverse_frequencies
from .attention import Attention, AttentionSpec
from .feed_forward import SwiGLU, SwiGLUSpec
from .block import ParallelBlock, PreNormBlock
from .sink_attention import SinkAttention, SinkAttentionSpec
from .moe import SigmoidMoE, SigmoidMoESpec
from .embedding import Embedding, EmbeddingSpec, Head, HeadSpec, PairEmbedding, PairEmbeddingSpec

__all__ = ["CacheNeed", "Part", "Runtime", "StepContext", "Linear", "RMSNorm", "RMSNormSpec", "Llama3Scaling",
           "NoPosition", "NoPositionSpec", "Rotary", "RotarySpec", "rotary_inverse_frequencies", "Attention",
           "AttentionSpec", "SwiGLU", "SwiGLUSpec", "PreNormBlock", "ParallelBlock", "SinkAttention", "SinkAttentionSpec", "SigmoidMoE", "SigmoidMoESpec",
           "DynamicTanh", "DynamicTanhSpec", "PairEmbedding", "PairEmbeddingSpec", "Embedding", "EmbeddingSpec", "Head", "HeadSpec"]
