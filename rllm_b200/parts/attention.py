"""Grouped-query attention over the paged cache, as a mixer part.

Order of operations as in the reference's Llama layer (src/model/registry/llama.rs:168-229):
q, k, v projections (here one product with the three weights stacked), optional bias,
rotation of q and k, write of k and v to the cache, attention with scale head_dim^-1/2
(src/gpu/cuda/shaders/attention.cu:336), output projection added to the residual stream.
A `window` limits each query to the last `window` keys
(src/gpu/cuda/shaders/attention.cu:337-338).
"""
from __future__ import annotations

from .base import KVCacheSpec, Param, Part, Source, register_part


class GQAttention(Part):
    graph_safe = True
    takes_deferred = True      # x goes to the backend's products as it comes

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, position: Part,
                 window: int | None = None, bias: bool = False, scale: float | None = None):
        if heads % kv_heads:
            raise ValueError(f"heads {heads} must be a multiple of kv_heads {kv_heads}")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} must be a multiple of 16, at most 256")
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.position, self.window, self.bias = position, window, bias
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.w_qkv = self.b_qkv = self.w_o = None

    @property
    def q_size(self):
        return self.heads * self.head_dim

    @property
    def kv_size(self):
        return self.kv_heads * self.head_dim

    def children(self):
        return [self.position]

    def params(self):
        H, Q, KV = self.hidden, self.q_size, self.kv_size
        ps = [Param("w_qkv", (Source("q_proj.weight", (Q, H)), Source("k_proj.weight", (KV, H)),
                              Source("v_proj.weight", (KV, H)))),
              Param("w_o", (Source("o_proj.weight", (H, Q)),))]
        if self.bias:
            # random-weights mode draws them like the matrices: a bias of zeros would hide a
            # kernel that drops it
            ps.append(Param("b_qkv", (Source("q_proj.bias", (Q,)), Source("k_proj.bias", (KV,)),
                                      Source("v_proj.bias", (KV,)))))
        return ps

    def cache_spec(self):
        return KVCacheSpec(self.kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, cache, residual):
        """x: normalised activations [T, hidden]; adds the mixer's output into `residual`."""
        be = ctx.backend
        if hasattr(self.position, "project_rotate_store"):
            qkv = self.position.project_rotate_store(x, self.w_qkv, self.b_qkv, ctx, cache, self.heads,
                                                     self.kv_heads)
        else:
            qkv = be.linear(x, self.w_qkv, bias=self.b_qkv)
            self.position.rotate_and_store(qkv, ctx, cache, self.heads, self.kv_heads)
        q = qkv[:, : self.q_size]
        attn = be.attention(q, cache, ctx, self.heads, self.scale, self.window)
        be.linear_residual(attn, self.w_o, residual)


register_part("mixer", "gqa", GQAttention)
