from .params import SamplingParams
from .sampler import Sampler, uniform

__all__ = ["Sampler", "SamplingParams", "uniform"]
