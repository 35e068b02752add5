"""Sampling parameters and the Philox generator; the samplers themselves are kernels (csrc/sampling.cu)."""
from .params import SamplingParams
from .philox import philox4x32, uniform

__all__ = ["SamplingParams", "philox4x32", "uniform"]
