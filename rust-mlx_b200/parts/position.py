"""Position encodings that an attention mixer can be given.

``RotaryEmbedding``: half-split rotation of the first ``rotary_dim`` numbers of a
head, inv_freq[j] = theta^(-2j / rotary_dim), angle = position * inv_freq[j]
(src/dense.rs:187-195 with traditional=false, scale 1; the pairing is spelled out
in kernels/text_rope.metal:3-14).  The table is made in float64 and held in
float32; the kernel forms the angle, its sine and cosine and the rotation in
float32.  ``NoPositionEncoding`` rotates nothing.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding


class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        self.theta = float(theta)
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self._table = (self.theta ** (-2.0 * j / max(self.rotary_dim, 1))).to(torch.float32)
        self.inv_freq = None

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.inv_freq = self._table.to(ctx.device).contiguous()

    def angles(self, batch):
        """[tokens, rotary_dim] float32: cosines then sines of the step's positions.  The same for every
        head and layer, so they are formed once per step and kept with the batch."""
        if self.rotary_dim == 0:
            return None
        cache = batch.per_step
        key = ("rope", id(self))
        if key not in cache:
            out = self.ctx.workspace.get(f"rope_table_{id(self)}", (batch.n_tokens, self.rotary_dim), torch.float32)
            self.ctx.ops.rope_table(batch.positions, self.inv_freq, self.rotary_dim, out)
            cache[key] = out
        return cache[key]


class NoPositionEncoding(PositionEncoding):
    graph_safe = True

    def angles(self, batch):
        return None

    rotary_dim = 0
    inv_freq = None
