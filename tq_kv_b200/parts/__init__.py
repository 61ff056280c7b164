"""Parts a layer is put together from, and their registries."""
from .attention import GQAttention
from .base import (FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, StepBatch, StepContext, WeightSpec,
                   float32_vector)
from .block import PrenormResidualBlock
from .embedding import LMHead, TokenEmbedding
from .feed_forward import SwiGLU
from .norm import RMSNorm
from .position import RotaryHalved
from .registry import make_block, make_part, part_kinds, register_block, register_part, unregister_part

register_part("rms_norm", RMSNorm, replace=True)
register_part("rotary_halved", RotaryHalved, replace=True)
register_part("gqa_attention", GQAttention, replace=True)
register_part("swiglu", SwiGLU, replace=True)
register_part("token_embedding", TokenEmbedding, replace=True)
register_part("lm_head", LMHead, replace=True)
register_block("prenorm_residual", PrenormResidualBlock, replace=True)

__all__ = ["FeedForward", "GQAttention", "LMHead", "Mixer", "Norm", "Part", "PositionEncoding",
           "PrenormResidualBlock", "RMSNorm", "RotaryHalved", "Runtime", "StepBatch", "StepContext", "SwiGLU",
           "TokenEmbedding", "WeightSpec", "float32_vector", "make_block", "make_part", "part_kinds",
           "register_block", "register_part", "unregister_part"]
