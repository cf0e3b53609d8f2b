"""A model: embedding, a set of blocks, the order in which they run, and the output head.

The order is data. `schedule` is a list of `LayerCall(block, cache_layer, writes)`:
a block may appear more than once (weight sharing), and a call may read the cache
layer that another call fills (`writes=False`). Cache layers are numbered per model;
the cache manager groups those with equal needs.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..parts.base import Part


@dataclass(frozen=True)
class LayerCall:
    block: int          # index into Model.blocks
    cache_layer: int    # which cache layer the mixer uses (-1: none)
    writes: bool = True  # False: read what another call wrote, write nothing


class Model:
    def __init__(self, config, embedding: Part, blocks: list[Part], schedule: list[LayerCall],
                 head: Part, prefix: str = "model."):
        self.config = config
        self.embedding, self.blocks, self.schedule, self.head = embedding, blocks, schedule, head
        self.prefix = prefix
        for call in schedule:
            if not 0 <= call.block < len(blocks):
                raise ValueError(f"schedule names block {call.block}, model has {len(blocks)}")
        self.num_cache_layers = 1 + max((c.cache_layer for c in schedule), default=-1)
        writers = {c.cache_layer for c in schedule if c.writes and c.cache_layer >= 0}
        for c in schedule:
            if c.cache_layer >= 0 and c.cache_layer not in writers:
                raise ValueError(f"cache layer {c.cache_layer} is read but never written")

    # -- structure
    def parts(self):
        yield from self.embedding.walk()
        for b in self.blocks:
            yield from b.walk()
        yield from self.head.walk()

    def cache_specs(self):
        """cache layer -> spec, from the block that writes it."""
        specs = {}
        for c in self.schedule:
            if c.cache_layer >= 0 and c.writes:
                spec = self.blocks[c.block].cache_spec()
                if c.cache_layer in specs and specs[c.cache_layer] != spec:
                    raise ValueError(f"cache layer {c.cache_layer} is written with two different specs")
                specs[c.cache_layer] = spec
        return [specs[i] for i in range(self.num_cache_layers)]

    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    def finalize(self, device, dtype):
        for p in self.parts():
            p.finalize(device, dtype)

    # -- running
    def forward(self, ctx, caches):
        """Run the step's tokens through every scheduled layer -> float32 [T, hidden]."""
        if hasattr(ctx, "per_forward"):
            ctx.per_forward.clear()
        h = self.embedding.forward(ctx)
        for call in self.schedule:
            cache = caches.layer_view(call.cache_layer, ctx, call.writes) if call.cache_layer >= 0 else None
            self.blocks[call.block].forward(h, ctx, cache)
        return h

    def logits(self, h, rows, ctx):
        return self.head.forward(h, rows, ctx)
