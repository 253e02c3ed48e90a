"""Greedy and temperature sampling."""
from .sampler import Sampler, SamplingParams, request_seed, seed_words

__all__ = ["Sampler", "SamplingParams", "request_seed", "seed_words"]
