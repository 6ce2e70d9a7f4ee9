"""Position encodings that an attention mixer can be given.

``RotaryEmbedding``: half-split rotation of the first ``rotary_dim`` numbers of a
head, inv_freq[j] = theta^(-2j / rotary_dim), angle = position * inv_freq[j]
(src/dense.rs:187-195 with traditional=false, scale 1; the pairing is spelled out
in kernels/text_rope.metal:3-14).  The table is made in float64 and held in
float32; the kernel forms the angle, its sine and cosine and the rotation in
float32.  ``NoPositionEncoding`` rotates nothing.

Scaled variants change the table only (the kernels take it as an argument) and, for
"yarn", the factor that attention scores are multiplied with; the reference's dense
model has neither (scale 1, src/dense.rs:187-195), so these follow the published
definitions:
  linear: inv_freq / factor (positions are read as position / factor).
  yarn:   pairs that turn often within the original context keep their frequency, pairs
          that turn less than once are divided by ``factor``, with a linear ramp over the
          pair index between them: the pair that makes b turns in L positions has index
          d(b) = rotary_dim * ln(L / (2 pi b)) / (2 ln theta); ramp from floor(d(beta_fast))
          to ceil(d(beta_slow)); q and k are each scaled by 0.1 ln(factor) + 1 (or
          ``attention_factor``), so scores by its square.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding


def scaled_inv_freq(inv_freq: torch.Tensor, theta: float, rotary_dim: int, scaling: dict | None) -> tuple:
    """(table, factor for q and k each) for a ``rope_scaling`` dictionary; float64 in, float64 out."""
    kind = None if not scaling else scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv_freq, 1.0
    factor = float(scaling.get("factor", 1.0))
    if not factor >= 1.0:
        raise ValueError(f"rope scaling factor must be at least 1, got {factor}")
    if kind == "linear":
        return inv_freq / factor, 1.0
    if kind == "yarn":
        original = float(scaling.get("original_max_position_embeddings") or 0)
        if original <= 0:
            raise ValueError("yarn scaling needs original_max_position_embeddings")
        fast, slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))

        def index_of(turns):
            return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
        half = rotary_dim // 2
        low = max(math.floor(index_of(fast)), 0)
        high = min(math.ceil(index_of(slow)), rotary_dim - 1)
        if high == low:
            high = low + 0.001
        ramp = ((torch.arange(half, dtype=torch.float64) - low) / (high - low)).clamp(0.0, 1.0)
        table = inv_freq / factor * ramp + inv_freq * (1.0 - ramp)
        given = scaling.get("attention_factor")
        return table, float(given) if given is not None else 0.1 * math.log(factor) + 1.0
    raise ValueError(f"rope scaling of type '{kind}' is not known (default, linear, yarn)")


class RotaryEmbedding(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None, scaling: dict | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        self.theta = float(theta)
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        table, qk_factor = scaled_inv_freq(self.theta ** (-2.0 * j / max(self.rotary_dim, 1)), self.theta,
                                           self.rotary_dim, scaling)
        self._table = table.to(torch.float32)
        self.score_scale = qk_factor * qk_factor   # what the mixer multiplies its score scale with
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
