"""Sampling: parameters, the counter-based uniform numbers and the device sampler."""
from .sampler import Sampler, SamplingParams, uniform

__all__ = ["Sampler", "SamplingParams", "uniform"]
