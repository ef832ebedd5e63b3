"""Sampling: greedy and temperature."""
from .sampler import Sampler, SamplingParams, uniform_for

__all__ = ["Sampler", "SamplingParams", "uniform_for"]
