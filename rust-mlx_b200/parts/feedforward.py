"""The dense feed-forward: down(silu(gate(x)) * up(x)) (src/dense.rs:293-298).

gate and up are one matrix product over the concatenated weights [gate; up]; the
pointwise part forms silu(gate) * up in float32 and rounds once, as the
reference's compiled graph does (src/compiled.rs:7-12).
"""
from __future__ import annotations

import torch

from .base import FeedForward, ParamSpec


class SwiGLUFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, width: int, inner: int):
        self.prefix, self.width, self.inner = prefix, int(width), int(inner)
        self.w_gate_up = self.w_down = None

    def param_specs(self):
        p = self.prefix
        return [ParamSpec(f"{p}.gate_proj.weight", (self.inner, self.width)),
                ParamSpec(f"{p}.up_proj.weight", (self.inner, self.width)),
                ParamSpec(f"{p}.down_proj.weight", (self.width, self.inner))]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        p = self.prefix
        self.w_gate_up = torch.cat([tensors.pop(f"{p}.gate_proj.weight"), tensors.pop(f"{p}.up_proj.weight")],
                                   dim=0).contiguous()
        self.w_down = tensors[f"{p}.down_proj.weight"].contiguous()

    def linear_weights(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, x, batch=None):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n = x.shape[0]
        gu = ws.get("gate_up", (n, 2 * self.inner), dt)
        ops.linear(x, self.w_gate_up, gu, ws, batch.status if batch is not None else None)
        act = ws.get("ffn_act", (n, self.inner), dt)
        ops.swiglu(gu, act)
        y = ws.get("ffn_out", (n, self.width), dt)
        ops.linear(act, self.w_down, y, ws, batch.status if batch is not None else None)
        return y
