"""Greedy, temperature and top-k sampling."""
from .samplers import Sampler, SamplingParams, uniform_from_counter

__all__ = ["Sampler", "SamplingParams", "uniform_from_counter"]
