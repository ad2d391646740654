"""Sampling: parameters, the per-request generator, and the device-side selection."""

from .mt19937_64 import MT19937_64
from .sampler import (GREEDY_TEMPERATURE, Sampler, SamplingLogprobs, SamplingParams, SamplingResult,
                      TokenLogprob)

__all__ = ["GREEDY_TEMPERATURE", "MT19937_64", "Sampler", "SamplingLogprobs", "SamplingParams", "SamplingResult",
           "TokenLogprob"]
