"""Greedy and temperature sampling on float32 logits.

Greedy is what the reference samples with (src/bin/infer.rs:57-59): argmax, the
lowest id on a tie (kernels/greedy_reduce.metal:10-14).  Temperature sampling
draws from softmax(logits / temperature) by inverting the cumulative sum with a
uniform number from ``rng.uniform``; temperature 0 is greedy.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .rng import uniform


class Sampler:
    def __init__(self, device):
        self.device = device

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        ops.sample(logits, None, None, out)
        return out

    def sample(self, logits: torch.Tensor, temperatures: list, seed: int, requests: list, steps: list,
               out: torch.Tensor | None = None) -> torch.Tensor:
        """One token per row: row r uses temperatures[r] and uniform(seed, requests[r], steps[r])."""
        n = logits.shape[0]
        if out is None:
            out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if not any(t > 0 for t in temperatures):
            ops.sample(logits, None, None, out)
            return out
        host = torch.tensor([list(map(float, temperatures)),
                             [uniform(seed, r, s) for r, s in zip(requests, steps)]], dtype=torch.float32)
        dev = host.to(logits.device)
        ops.sample(logits, dev[0].contiguous(), dev[1].contiguous(), out)
        return out
