from .params import SamplingParams
from .rng import uniform
from .sampler import Sampler

__all__ = ["SamplingParams", "uniform", "Sampler"]
