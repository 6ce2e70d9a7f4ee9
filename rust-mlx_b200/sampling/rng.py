"""Uniform numbers for sampling, keyed by (seed, request, step).

A counter-based generator: the number for a request's n-th token depends on the
seed, the request's index and n only, not on which other requests share the
batch or on how the run was scheduled.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    """The finaliser of SplitMix64."""
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, request: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32)."""
    z = _mix(seed & _MASK)
    z = _mix(z ^ (request & _MASK))
    z = _mix(z ^ (step & _MASK))
    return (z >> 40) / float(1 << 24)
