"""RMSNorm fused with the residual add.

RMSNorm(v; w, eps) = v * rsqrt(mean(v^2) + eps) * w over the last axis, with the
plain weight (src/dense.rs:382,385-391).  The residual stream is float32; the
kernel adds the pending delta, stores the sum back and writes the normalised rows
in the compute dtype.  The weight is held in float32 (exact for a bfloat16
checkpoint) so both paths read the same numbers.
"""
from __future__ import annotations

from .base import Norm, ParamSpec


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, name: str, width: int, eps: float):
        self.name, self.width, self.eps = name, int(width), float(eps)
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.width,), "norm", "float32")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = tensors[self.name].contiguous()

    def forward(self, h, delta):
        x = self.ctx.workspace.get("norm_out", (h.shape[0], self.width), self.ctx.dtype)
        self.ctx.ops.add_rmsnorm(h, delta, self.weight, self.eps, x)
        return h, x

    def forward_rows(self, h, delta, rows):
        x = self.ctx.workspace.get("norm_rows_out", (rows.shape[0], self.width), self.ctx.dtype)
        self.ctx.ops.add_rmsnorm(h, delta, self.weight, self.eps, x, rows=rows)
        return x
