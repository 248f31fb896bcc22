from .params import GenerateOptions, SamplingParams
from .sampler import Sampler, uniform24

__all__ = ["GenerateOptions", "SamplingParams", "Sampler", "uniform24"]
