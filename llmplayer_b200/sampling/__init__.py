"""Samplers: options in the reference's terms, per-request state, the device kernel's caller."""
from .java_random import JavaRandom
from .params import SamplerConfig, SamplingParams
from .sampler import BatchSampler, SequenceSampler

__all__ = ["BatchSampler", "JavaRandom", "SamplerConfig", "SamplingParams", "SequenceSampler"]
