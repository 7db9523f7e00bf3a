"""The parts layers are put together from: norm, position encoding, mixer, feed-forward, block,
embedding and head.  Importing this package registers the built-in kinds."""
from .base import CacheNeed, Part, Runtime, StepContext
from .linear import Linear
from .norm import DynamicTanh, DynamicTanhSpec, PostNormed, PostRMSNorm, PostRMSNormSpec, RMSNorm, RMSNormSpec
from .position import Llama3Scaling, NoPosition, NoPositionSpec, Rotary, RotarySpec, rotary_inverse_frequencies
from .attention import Attention, AttentionSpec
from .feed_forward import BiasedMLP, BiasedMLPSpec, SwiGLU, SwiGLUSpec
from .block import ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock
from .sink_attention import SinkAttention, SinkAttentionSpec
from .moe import SigmoidMoE, SigmoidMoESpec
from .embedding import Embedding, EmbeddingSpec, Head, HeadSpec, PairEmbedding, PairEmbeddingSpec, ScaledEmbedding, ScaledEmbeddingSpec
from .mamba2 import Mamba2, Mamba2Spec
from .gated_delta import GatedDelta, GatedDeltaSpec
from .sigmoid_attention import SigmoidAttention, SigmoidAttentionSpec
from .parallel_mixers import ParallelMixers, ParallelMixersSpec
from .filter import ShortConv, ShortConvSpec
from .latent_attention import LatentAttention, LatentAttentionSpec
from .hgrn2 import Hgrn2, Hgrn2Spec
from .wkv import Wkv, WkvSpec
from .stream import ConcatProjection, ConcatProjectionSpec
from .normed_attention import NormedAttention, NormedAttentionSpec

__all__ = ["CacheNeed", "Part", "Runtime", "StepContext", "Linear", "RMSNorm", "RMSNormSpec", "Llama3Scaling",
           "NoPosition", "NoPositionSpec", "Rotary", "RotarySpec", "rotary_inverse_frequencies", "Attention",
           "AttentionSpec", "SwiGLU", "SwiGLUSpec", "PreNormBlock", "ParallelBlock", "SinkAttention", "SinkAttentionSpec", "SigmoidMoE", "SigmoidMoESpec",
           "DynamicTanh", "DynamicTanhSpec", "PairEmbedding", "PairEmbeddingSpec", "Embedding", "EmbeddingSpec", "Head", "HeadSpec",
           "PostNormed", "PostRMSNorm", "PostRMSNormSpec", "BiasedMLP", "BiasedMLPSpec", "SandwichBlock", "ScaledEmbedding",
           "ScaledEmbeddingSpec", "Mamba2", "Mamba2Spec", "GatedDelta", "GatedDeltaSpec", "SigmoidAttention", "SigmoidAttentionSpec",
           "ParallelMixers", "ParallelMixersSpec", "ShortConv", "ShortConvSpec", "LatentAttention", "LatentAttentionSpec", "Hgrn2",
           "Hgrn2Spec", "Wkv", "WkvSpec", "ConcatProjection", "ConcatProjectionSpec", "NormedAttention", "NormedAttentionSpec",
           "PostNormBlock"]
