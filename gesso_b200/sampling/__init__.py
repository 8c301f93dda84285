"""Sampling: greedy, temperature, nucleus."""
from .sampler import SamplingParams, SplitMix64, greedy_host, sample_host, select_tokens

__all__ = ["SamplingParams", "SplitMix64", "greedy_host", "sample_host", "select_tokens"]
