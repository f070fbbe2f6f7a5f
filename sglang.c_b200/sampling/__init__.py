from .params import SamplingParams
from .rng import mix64, request_stream, uniform
from .sampler import Sampler

__all__ = ["SamplingParams", "Sampler", "mix64", "request_stream", "uniform"]
