"""Rotary position encoding as a part: a table of inverse frequencies, made once on the
host in float64 and kept as float32; the rotation itself runs inside the kernel that
also writes K and V to the cache.

Plain rule f_i = theta^(-2i/d): src/gpu/cuda/shaders/rope.cu:62-66 of the reference. A
model's own rule (`rope_scaling.rope_type`) is looked up by name in `rope_rules`.
"""
from __future__ import annotations

import torch

from .base import Part, register_part
from .rope_rules import rope_rule


def inverse_frequencies(rot_dim: int, theta: float, scaling=None) -> list[float]:
    """The rot_dim/2 inverse frequencies in float64, the scaling rule applied. `scaling`: None, or
    an object with `rope_type` and `to_dict()` (the rule's parameters)."""
    freqs = [float(theta) ** (-2.0 * i / rot_dim) for i in range(rot_dim // 2)]
    if scaling is not None and scaling.rope_type != "default":
        freqs = list(rope_rule(scaling.rope_type)(freqs, scaling.to_dict()))
        if len(freqs) != rot_dim // 2:
            raise ValueError(f"rope rule {scaling.rope_type!r} returned {len(freqs)} frequencies for {rot_dim // 2}")
    return freqs


class RotaryEmbedding(Part):
    """Rotates pairs (i, i + rot_dim/2) of each head by position * f_i."""
    graph_safe = True

    def __init__(self, head_dim: int, theta: float, scaling=None, rot_dim: int | None = None):
        self.head_dim = head_dim
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rotary width {self.rot_dim} must be even and <= head_dim {head_dim}")
        self.theta, self.scaling = float(theta), scaling
        self.inv_freq = None
        # layers with the same rule share one table of angles per step
        self.table_key = ("rope", self.rot_dim, self.theta, repr(scaling))

    def finalize(self, device, dtype):
        f = inverse_frequencies(self.rot_dim, self.theta, self.scaling)
        self.inv_freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device)

    def project_rotate_store(self, x, w_qkv, bias, ctx, cache, nh, nkv):
        """qkv = x w_qkv^T (+ bias) with q and k rotated and k, v written into the layer's pages:
        the projection and this part's work in one kernel where the backend can."""
        return ctx.backend.qkv_rope_cache_write(x, w_qkv, bias, ctx.positions, self.inv_freq, cache, nh, nkv,
                                                self.head_dim, self.rot_dim, ctx=ctx, key=self.table_key)

    def rotate_and_store(self, qkv, ctx, cache, nh, nkv):
        """Rotate q (in place) and k of `qkv`, and write k, v into the layer's pages."""
        ctx.backend.rope_cache_write(qkv, ctx.positions, self.inv_freq, cache, nh, nkv,
                                     self.head_dim, self.rot_dim, ctx=ctx, key=self.table_key)


register_part("position", "rope", RotaryEmbedding)
