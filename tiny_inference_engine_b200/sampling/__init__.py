"""Sampling parameters, the Philox generator, and the samplers."""
from .params import SamplingParams
from .philox import philox4x32, uniform
from .sampler import sample_host

__all__ = ["SamplingParams", "philox4x32", "uniform", "sample_host"]
