"""The dense feed-forward: down(silu(gate(x)) * up(x)) (src/dense.rs:293-298).

gate and up are one matrix product over fused weights: blocks of 64 gate rows each
followed by their 64 up rows (plain concatenation when the width is no multiple of
64), so that a tile of 128 output rows of the tensor-core product holds gates and
their ups and can form silu(gate) * up in its epilogue.  Each output row is the same
dot product as with separate weights.  The pointwise part is formed in float32 and
rounded once, as the reference's compiled graph does (src/compiled.rs:7-12).
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
        gate, up = tensors.pop(f"{p}.gate_proj.weight"), tensors.pop(f"{p}.up_proj.weight")
        self.block = 64 if self.inner % 64 == 0 else 0
        if self.block:
            g = gate.view(self.inner // 64, 64, self.width)
            u = up.view(self.inner // 64, 64, self.width)
            self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.inner, self.width).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[f"{p}.down_proj.weight"].contiguous()

    def linear_weights(self):
        return [self.w_gate_up, self.w_down]

    def gate_up_weights(self):
        return [self.w_gate_up] if self.block else []

    def forward(self, x, batch=None):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n = x.shape[0]
        status = batch.status if batch is not None else None
        act = ws.get("ffn_act", (n, self.inner), dt)
        if self.block and dt == torch.bfloat16 and ops.prefers_fused_swiglu(n, 2 * self.inner, self.width):
            ops.gemm_tcgen05(x, self.w_gate_up, act, ws, status, dependent=ops.dependent_launch, swiglu=True)
        else:
            gu = ws.get("gate_up", (n, 2 * self.inner), dt)
            ops.linear(x, self.w_gate_up, gu, ws, status)
            ops.swiglu(gu, act, self.block)
        if self.ctx.tap is not None:
            self.ctx.tap("ffn_act", act)
        y = ws.get("ffn_out", (n, self.width), dt)
        ops.linear(act, self.w_down, y, ws, status)
        return y
