"""Sampling: parameters, the host random stream, and the GPU sampler."""
from .params import SamplingParams, XorShift64Star
from .sampler import Sampler

__all__ = ["SamplingParams", "XorShift64Star", "Sampler"]
