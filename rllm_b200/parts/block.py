"""How a layer's parts are arranged. Pre-norm residual block, the reference's Llama layer
order (src/model/registry/llama.rs:163-245): h += mixer(norm(h)); h += ffn(norm(h))."""
from __future__ import annotations

from .base import Part, register_part


class PreNormBlock(Part):
    """`names` maps the four parts to their checkpoint sub-prefixes."""
    graph_safe = True

    def __init__(self, mixer_norm: Part, mixer: Part, ffn_norm: Part, ffn: Part,
                 names=("input_layernorm.", "self_attn.", "post_attention_layernorm.", "mlp.")):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.names = names

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def set_prefix(self, prefix: str):
        self.prefix = prefix
        for part, sub in zip(self.children(), self.names):
            part.prefix = prefix + sub
            for c in part.children():
                if not c.prefix:
                    c.prefix = part.prefix

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, h, ctx, cache):
        """h: float32 residual stream [T, hidden], updated in place."""
        self.mixer.forward(self._norm(self.mixer_norm, self.mixer, h, ctx), ctx, cache, h)
        self.ffn.forward(self._norm(self.ffn_norm, self.ffn, h, ctx), ctx, h)
        return h

    @staticmethod
    def _norm(norm, consumer, h, ctx):
        """A consumer that hands its input straight to the backend's products (`takes_deferred`)
        gets the norm in deferred form, so that it can run inside the first product."""
        if getattr(consumer, "takes_deferred", False) and hasattr(norm, "deferred"):
            return norm.deferred(h, ctx)
        return norm.forward(h, ctx)


register_part("block", "prenorm", PreNormBlock)
