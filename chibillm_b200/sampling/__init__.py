"""Sampling: greedy and temperature."""
from .sampler import PendingTokens, Sampler, SamplingParams, uniform_for

__all__ = ["PendingTokens", "Sampler", "SamplingParams", "uniform_for"]
