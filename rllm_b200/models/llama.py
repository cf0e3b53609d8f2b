"""Llama (LlamaForCausalLM) assembled from parts. Layer order and tensor names as in the
reference (src/model/registry/llama.rs:163-245; names: src/model/loader/mod.rs:794-798,
1436-1464, 1558-1578, 748, 693-702). Everything numeric comes from the configuration."""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.llama import LlamaConfig
from ..parts import GQAttention, PreNormBlock, RMSNorm, RotaryEmbedding, SwiGLU, make_part
from .model import LayerCall, Model


def build_llama(cfg: LlamaConfig) -> Model:
    prefix = "model."
    emb = make_part("embedding", "table", vocab=cfg.vocab_size, hidden=cfg.hidden_size)
    emb.prefix = prefix
    blocks = []
    for i in range(cfg.num_hidden_layers):
        rope = RotaryEmbedding(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling)
        block = PreNormBlock(
            RMSNorm(cfg.hidden_size, cfg.rms_norm_eps),
            GQAttention(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                        cfg.head_dim, rope, window=cfg.layer_window(i), bias=cfg.attention_bias),
            RMSNorm(cfg.hidden_size, cfg.rms_norm_eps),
            SwiGLU(cfg.hidden_size, cfg.intermediate_size))
        block.set_prefix(f"{prefix}layers.{i}.")
        blocks.append(block)
    final_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
    final_norm.prefix = prefix + "norm."
    head = make_part("head", "linear", vocab=cfg.vocab_size, hidden=cfg.hidden_size, norm=final_norm,
                     tied_to=emb if cfg.tie_word_embeddings else None)
    head.prefix = "lm_head."
    schedule = [LayerCall(i, i, True) for i in range(cfg.num_hidden_layers)]
    return Model(cfg, emb, blocks, schedule, head, prefix)


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama, model_types=("llama",))
