"""Greedy and temperature sampling."""
from .sampler import Sampler, SamplingError, SamplingParams

__all__ = ["Sampler", "SamplingError", "SamplingParams"]
