"""RMS norm: out = x / sqrt(mean(x^2) + eps) * gain, in float32.

Reference: inference/RMSNorm.java:17-35, tensor/ScalarOps.java:26-35,
src/main/resources/kernels/cuda/rmsnorm.cu:6-46. The gain is used as stored.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import NORMS, Part, Runtime
from .specs import GAIN, NormSpec, TensorSpec


class RMSNorm(Part):
    capture_safe = True
    fusable_rms = True      # a product that adds into the residual stream may write this norm on the way

    def __init__(self, spec: NormSpec):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.spec.weight: TensorSpec((self.spec.size,), GAIN)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        self.weight = runtime.gain(tensors[self.spec.weight])

    def apply(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None,
              add: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out[r] = norm(x[rows[r]])``; ``add`` is summed into ``x`` first (in place);
        ``clear`` is a float32 buffer zeroed on the side."""
        return ops.rmsnorm(x, self.weight, self.spec.eps, out, rows=rows, add=add, clear=clear)


NORMS.register("rmsnorm", RMSNorm)
