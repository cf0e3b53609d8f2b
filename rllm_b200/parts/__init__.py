from .base import (KVCacheSpec, LayerCache, Param, Part, Source, StateSpec, make_part,
                   register_part, registered_parts)
from .norm import RMSNorm
from .rope import RotaryEmbedding, inverse_frequencies
from .attention import GQAttention
from .ffn import SwiGLU
from .block import PreNormBlock
from .embedding import Embedding, OutputHead

__all__ = ["KVCacheSpec", "LayerCache", "Param", "Part", "Source", "StateSpec", "make_part",
           "register_part", "registered_parts", "RMSNorm", "RotaryEmbedding",
           "inverse_frequencies", "GQAttention", "SwiGLU", "PreNormBlock", "Embedding",
           "OutputHead"]
