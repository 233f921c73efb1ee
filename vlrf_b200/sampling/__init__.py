from .params import SamplingParams
from .rng import request_key, uniform01
from .sampler import RowSampler

__all__ = ["SamplingParams", "request_key", "uniform01", "RowSampler"]
