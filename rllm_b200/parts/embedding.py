"""Token embedding and output head. Embedding is a row copy with no scaling
(src/gpu/cuda/shaders/embed.cu:24-59); the head is final norm, then a product with
`lm_head.weight`, or with the embedding table when the two are tied
(src/model/primitives.rs:124-143, 1467; src/model/loader/mod.rs:693-702). Logits are
float32 and are computed only for the rows that were asked for."""
from __future__ import annotations

from .base import Param, Part, Source, register_part


class Embedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, name: str = "embed_tokens.weight"):
        self.vocab, self.hidden, self.name = vocab, hidden, name
        self.table = None

    def params(self):
        return [Param("table", (Source(self.name, (self.vocab, self.hidden)),))]

    def forward(self, ctx):
        return ctx.backend.embed(ctx.token_ids, self.table, err=ctx.extras.get("err_flag"))


class OutputHead(Part):
    """`tied_to`: the Embedding whose table doubles as the output matrix, or None."""
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, norm: Part, tied_to: Embedding | None,
                 name: str = "weight"):
        self.vocab, self.hidden, self.norm, self.tied_to, self.name = vocab, hidden, norm, tied_to, name
        self.weight = None

    def children(self):
        return [self.norm]

    def params(self):
        if self.tied_to is not None:
            return []
        return [Param("weight", (Source(self.name, (self.vocab, self.hidden)),))]

    def matrix(self):
        return self.tied_to.table if self.tied_to is not None else self.weight

    def forward(self, h, rows, ctx):
        """h: float32 [T, hidden]; rows: int32 device vector of the wanted rows -> [R, vocab]."""
        if hasattr(self.norm, "deferred"):
            n = self.norm.deferred(h, ctx, rows)      # gather, norm and product may be one kernel
        else:
            n = self.norm.forward(ctx.backend.gather_rows(h, rows), ctx)
        return ctx.backend.linear_f32(n, self.matrix())


register_part("embedding", "table", Embedding)
register_part("head", "linear", OutputHead)
