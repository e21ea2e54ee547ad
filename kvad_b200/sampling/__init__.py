"""Sampling: options, per-request streams, the host statement of the rule."""
from .sampler import RequestSampler, SamplingParams, Xorshift64Star, argmax, sample_host, shortlist

__all__ = ["RequestSampler", "SamplingParams", "Xorshift64Star", "argmax", "sample_host", "shortlist"]
