"""SwiGLU feed-forward as a part: down(silu(gate x) * (up x)), added to the residual
stream. Formula: src/gpu/cuda/shaders/moe.cu:141-146 and src/model/primitives.rs:557-585
of the reference. Gate and up weights are stacked so that one product yields both."""
from __future__ import annotations

from .base import Param, Part, Source, register_part


class SwiGLU(Part):
    graph_safe = True
    takes_deferred = True      # x goes to the backend's products as it comes

    def __init__(self, hidden: int, intermediate: int):
        self.hidden, self.intermediate = hidden, intermediate
        self.w_gate_up = self.w_down = None

    def params(self):
        H, I = self.hidden, self.intermediate
        return [Param("w_gate_up", (Source("gate_proj.weight", (I, H)), Source("up_proj.weight", (I, H)))),
                Param("w_down", (Source("down_proj.weight", (H, I)),))]

    def forward(self, x, ctx, residual):
        be = ctx.backend
        act = be.linear_swiglu(x, self.w_gate_up)
        be.linear_residual(act, self.w_down, residual)


register_part("ffn", "swiglu", SwiGLU)
