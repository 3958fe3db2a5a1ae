from .base import (Block, BuildContext, FeedForward, KVCacheNeed, Mixer, Norm, Part, PositionEncoding, StateNeed,
                   TensorSpec, make_part, prefixed, register_part, take, unregister_part)
from .attention import GQAttention
from .block import OutputNormBlock, ParallelBlock, PreNormBlock
from .embedding import HashedBigramEmbedding, LMHead, TokenEmbedding
from .latent_attention import LatentAttention
from .linear_attention import GatedDeltaRule, GatedLinearAttention, ParallelMixer
from .mlp import PlainMLP, SwiGLUMLP
from .moe import RoutedExperts
from .norm import RMSNorm
from .rglru import RGLRUMixer
from .rope import NoPosition, RotaryPosition

for _kind, _cls in (("rmsnorm", RMSNorm), ("rope", RotaryPosition), ("no_position", NoPosition),
                    ("gqa_attention", GQAttention), ("swiglu_mlp", SwiGLUMLP), ("prenorm_block", PreNormBlock),
                    ("token_embedding", TokenEmbedding), ("lm_head", LMHead), ("latent_attention", LatentAttention),
                    ("rglru", RGLRUMixer), ("routed_experts", RoutedExperts), ("outnorm_block", OutputNormBlock),
                    ("plain_mlp", PlainMLP), ("gated_linear_attention", GatedLinearAttention),
                    ("gated_delta_rule", GatedDeltaRule), ("parallel_mixer", ParallelMixer),
                    ("parallel_block", ParallelBlock), ("hashed_bigram_embedding", HashedBigramEmbedding)):
    register_part(_kind, _cls, replace=True)

__all__ = [
    "Block", "BuildContext", "FeedForward", "GQAttention", "GatedDeltaRule", "GatedLinearAttention", "HashedBigramEmbedding",
    "OutputNormBlock", "ParallelBlock",
    "ParallelMixer", "PlainMLP", "KVCacheNeed", "LMHead", "LatentAttention", "Mixer",
    "NoPosition", "Norm", "Part", "PositionEncoding", "PreNormBlock", "RGLRUMixer", "RMSNorm", "RotaryPosition",
    "RoutedExperts", "StateNeed", "SwiGLUMLP", "TensorSpec",
    "TokenEmbedding", "make_part", "prefixed", "register_part", "take", "unregister_part",
]
