"""Sampler options, with the reference's names, meanings and defaults.

Reference: sampler/SamplerConfig.java:15-21 (defaults: temperature 0.7, top-k 40,
top-p 0.9, repetition penalty 1.1, seed from the clock; min-p, mirostat and DRY
off), :83-85 (``greedy()``: temperature 0, top-k 1, top-p 1, penalty 1, seed 0).
Pipeline order (sampler/CompositeSampler.java:33-120): DRY penalty, repetition
penalty, greedy if temperature is 0, else 1/temperature, top-k, softmax, min-p,
top-p, then mirostat v2 or a multinomial draw.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field, replace

from ..errors import RequestError


def _clock_seed() -> int:
    return time.time_ns()


@dataclass(frozen=True)
class SamplerConfig:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.1
    seed: int = field(default_factory=_clock_seed)
    min_p: float = 0.0
    mirostat: int = 0              # 0 = off, 2 = mirostat v2
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    dry_multiplier: float = 0.0    # 0 = off
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_range: int = 1024

    def __post_init__(self):
        if self.temperature < 0:
            raise RequestError(f"temperature must not be negative, got {self.temperature}")
        if self.repetition_penalty <= 0:
            raise RequestError(f"repetition_penalty must be positive, got {self.repetition_penalty}")
        if self.mirostat not in (0, 2):
            raise RequestError(f"mirostat must be 0 (off) or 2, got {self.mirostat}")
        if not 0 <= self.min_p <= 1:
            raise RequestError(f"min_p must lie in [0, 1], got {self.min_p}")

    @classmethod
    def greedy(cls) -> "SamplerConfig":
        return cls(temperature=0.0, top_k=1, top_p=1.0, repetition_penalty=1.0, seed=0)

    def with_seed(self, seed: int) -> "SamplerConfig":
        return replace(self, seed=seed)

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0


SamplingParams = SamplerConfig
