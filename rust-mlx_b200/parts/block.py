"""How a mixer, a feed-forward and their norms are arranged in a layer.

``PreNormBlock``: h += mixer(norm1(h)); h += ffn(norm2(h)) (src/dense.rs:380-390).
The residual stream is float32.  A block receives the stream together with a
pending delta (the previous block's last output, not yet added) so that every
add is fused with the norm that follows it; it returns the stream and its own
pending delta.
"""
from __future__ import annotations

from .base import Part


class PreNormBlock(Part):
    graph_safe = True

    def __init__(self, norm1, mixer, norm2, ffn):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    def children(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def cache_specs(self):
        return self.mixer.cache_specs()

    def forward(self, h, pending, batch, cache):
        tap = self.ctx.tap
        h, x = self.norm1.forward(h, pending)
        if tap is not None:
            tap("residual", h)      # the stream as this block finds it: everything before it has been added
            tap("norm1", x)
        a = self.mixer.forward(x, batch, cache)
        if tap is not None:
            tap("mixer_out", a)
        h, x = self.norm2.forward(h, a)
        if tap is not None:
            tap("norm2", x)
        m = self.ffn.forward(x, batch)
        if tap is not None:
            tap("ffn_out", m)
        return h, m
