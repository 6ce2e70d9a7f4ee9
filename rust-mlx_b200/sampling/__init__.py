"""Choosing tokens: the kernel is ``ops.sample`` (greedy and temperature rows in one launch); the uniform numbers of
temperature sampling come from ``rng.uniform``, keyed by (seed, request, step)."""
from .rng import uniform

__all__ = ["uniform"]
