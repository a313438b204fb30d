"""Position encodings of a mixer's queries and keys.

A position part owns the rule. It offers it in one of two forms: ``rotation()`` returns an
:class:`llmplayer_b200.kernels.ops.Rotation` when the rule is a rotation of feature pairs by
position x frequency, which the kernels that prepare queries and keys apply on the way; a part
whose rule is anything else returns None there and implements ``apply(ctx, qkv, num_heads=,
num_kv_heads=, head_dim=)``, which changes the query and key heads of the float32 projection
``qkv`` [T, (H + 2G) * hd] (or [T, H * hd] for a layer without keys of its own) in place, reading
the tokens' positions from ``ctx.positions``; the mixer then runs its kernels without rotation.

Rotary encoding: the per-pair frequencies the kernels rotate by.

Reference: inference/RoPE.java:80-105. f_i = 1 / theta^(2i / rotary_dim) is
computed in double and rounded to float32 (:83); a per-pair divisor may follow
(:85-87), which for "llama3" scaling is what the model file's converter derives
from the wavelength rule implemented here. The angle position * f_i is a
float32 product (:101), evaluated inside the kernel that rotates.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..errors import ConfigError
from ..kernels import ops
from .base import POSITIONS, Part, Runtime
from .specs import PositionSpec


def inverse_frequencies(spec: PositionSpec) -> torch.Tensor:
    if spec.rotary_dim <= 0 or spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim:
        raise ConfigError(f"rotary width {spec.rotary_dim} does not fit a head of {spec.head_dim}")
    if not spec.theta > 0:
        raise ConfigError(f"rope theta must be positive, got {spec.theta}")
    freqs = []
    s = spec.scaling
    for i in range(spec.rotary_dim // 2):
        f = 1.0 / math.pow(spec.theta, 2.0 * i / spec.rotary_dim)
        if s is not None:
            wavelength = 2.0 * math.pi / f
            short = s.original_max_position / s.high_freq_factor
            long = s.original_max_position / s.low_freq_factor
            if wavelength > long:
                f = f / s.factor
            elif wavelength >= short:
                blend = (s.original_max_position / wavelength - s.low_freq_factor) / (
                    s.high_freq_factor - s.low_freq_factor)
                f = (1.0 - blend) * f / s.factor + blend * f
        freqs.append(f)
    return torch.tensor(freqs, dtype=torch.float64).to(torch.float32)


class Rotary(Part):
    """Rotation of query and key pairs by position x frequency: a rule the kernels apply themselves."""
    capture_safe = True

    def __init__(self, spec: PositionSpec):
        if spec.pairing not in ("split_half", "interleaved"):
            raise ConfigError(f"unknown rotary pairing {spec.pairing!r}")
        self.spec = spec
        self._rotation: Optional[ops.Rotation] = None

    def load(self, tensors, runtime: Runtime) -> None:
        super().load(tensors, runtime)
        # layers with equal specifications share one table of frequencies (and, per step, one table of angles)
        inv_freq = runtime.shared(("rotary", self.spec), lambda: inverse_frequencies(self.spec).to(runtime.device))
        self._rotation = ops.Rotation(inv_freq, self.spec.rotary_dim, self.spec.pairing == "interleaved")

    def rotation(self) -> Optional[ops.Rotation]:
        return self._rotation

    def apply(self, ctx, qkv, *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        raise ConfigError("a rotary encoding is applied by the kernels that take its rotation()")


class NoPosition(Part):
    """Queries and keys are used as projected."""
    capture_safe = True

    def __init__(self, spec: PositionSpec):
        self.spec = spec

    def rotation(self) -> Optional[ops.Rotation]:
        return ops.NO_ROTATION

    def apply(self, ctx, qkv, *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        pass


POSITIONS.register("rope", Rotary)
POSITIONS.register("none", NoPosition)
