"""Sampling parameters and the device sampler."""
from .params import SamplingParams
from .sampler import Sampler, SamplingRow

__all__ = ["SamplingParams", "Sampler", "SamplingRow"]
