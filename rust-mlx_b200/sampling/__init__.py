from .rng import uniform
from .sampler import Sampler

__all__ = ["Sampler", "uniform"]
