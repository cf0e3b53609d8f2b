from .base import (CacheKind, KVCacheSpec, LayerCache, Param, Part, Source, StateSpec, cache_kind_of,
                   make_part, register_cache_kind, register_part, registered_parts)
from .rope_rules import register_rope_rule, registered_rope_rules
from .norm import RMSNorm
from .rope import RotaryEmbedding, inverse_frequencies
from .attention import GQAttention
from .ffn import SwiGLU
from .block import PreNormBlock
from .embedding import Embedding, OutputHead

__all__ = ["CacheKind", "cache_kind_of", "register_cache_kind", "register_rope_rule", "registered_rope_rules",
           "KVCacheSpec", "LayerCache", "Param", "Part", "Source", "StateSpec", "make_part",
           "register_part", "registered_parts", "RMSNorm", "RotaryEmbedding",
           "inverse_frequencies", "GQAttention", "SwiGLU", "PreNormBlock", "Embedding",
           "OutputHead"]
