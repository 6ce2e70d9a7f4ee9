"""Token embedding and the output head.

h = embed_tokens.weight[ids] (src/weights.rs:203-204); logits = x . lm_head^T, or
x . embed_tokens^T when the head is tied (src/dense.rs:358-362,392-396).  Logits
come out in float32 in every run, and only for the rows that are asked for.
"""
from __future__ import annotations

import torch

from .base import ParamSpec, Part


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, name: str, vocab: int, width: int):
        self.name, self.vocab, self.width = name, int(vocab), int(width)
        self.weight = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.vocab, self.width), "embedding")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = tensors[self.name].contiguous()

    def forward(self, ids, batch=None):
        """Rows of the table for ``ids``; where the batch says so (``from_last``) a token's id is the one the last
        step's sampling left on the device for its sequence."""
        h = self.ctx.workspace.get("residual", (ids.shape[0], self.width), torch.float32)
        if batch is not None and batch.last_tokens is not None:
            self.ctx.ops.embedding(ids, self.weight, h, batch.from_last, batch.seq_index, batch.slots, batch.last_tokens)
        else:
            self.ctx.ops.embedding(ids, self.weight, h)
        return h


class OutputHead(Part):
    graph_safe = True

    """``name`` of its own weight, or ``tied_to`` an embedding whose table it reads."""

    def __init__(self, vocab: int, width: int, name: str | None = None, tied_to: TokenEmbedding | None = None):
        if (name is None) == (tied_to is None):
            raise ValueError("an output head has either its own weight or a tied embedding")
        self.name, self.tied_to, self.vocab, self.width = name, tied_to, int(vocab), int(width)
        self.weight = None

    def param_specs(self):
        return [] if self.name is None else [ParamSpec(self.name, (self.vocab, self.width), "linear")]

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        self.weight = self.tied_to.weight if self.name is None else tensors[self.name].contiguous()

    def linear_weights(self):
        return [self.weight]

    def forward(self, x, batch=None):
        logits = self.ctx.workspace.get("logits", (x.shape[0], self.vocab), torch.float32)
        self.ctx.ops.linear(x, self.weight, logits, self.ctx.workspace, batch.status if batch is not None else None)
        return logits
