"""Scratch tensors that kernels hand to one another, kept between steps.

``get(name, shape, dtype)`` returns a view of a buffer that lives as long as the
engine; a buffer grows when a larger shape is asked for, unless the workspace is
frozen (while a CUDA graph that holds its addresses exists).
"""
from __future__ import annotations

import math

import torch


class Workspace:
    def __init__(self, device):
        self.device = device
        self.buffers = {}
        self.views = {}       # (name, dtype, shape) -> the view handed out last time (a step asks for hundreds)
        self.frozen = False
        self.generation = 0   # counts reallocations: who holds addresses compares it

    def get(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        view = self.views.get((name, dtype, shape))
        if view is not None:
            return view
        numel = math.prod(shape)
        key = (name, dtype)
        buf = self.buffers.get(key)
        if buf is None or buf.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name} would have to grow to {numel} while frozen")
            if buf is not None:
                self.generation += 1
                self.views = {k: v for k, v in self.views.items() if k[:2] != key}
            buf = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self.buffers[key] = buf
        if len(self.views) > 4096:
            self.views.clear()
        view = self.views[(name, dtype, shape)] = buf[:numel].view(shape)
        return view

    def get_zeroed(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        """Like ``get``, but the buffer is zero when it is first made (or made again, larger);
        whoever uses it leaves it zero."""
        numel = math.prod(shape)
        key = (name, dtype)
        buf = self.buffers.get(key)
        if buf is None or buf.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name} would have to grow to {numel} while frozen")
            if buf is not None:
                self.generation += 1
                self.views = {k: v for k, v in self.views.items() if k[:2] != key}
            buf = torch.zeros(max(numel, 1), dtype=dtype, device=self.device)
            self.buffers[key] = buf
        return buf[:numel].view(shape)

    def reserve(self, name: str, shape: tuple, dtype: torch.dtype) -> None:
        self.get(name, shape, dtype)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.buffers.values())
