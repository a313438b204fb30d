"""Dense gated feed-forward: residual += down(silu(gate x) * (up x)).

Gate and up are held as one stacked matrix so that one product yields both and
the activation is applied where the sums are formed.

Reference: inference/SwiGLUFFN.java:36-67, tensor/ScalarOps.java:69-73,
src/main/resources/kernels/cuda/silu_mul.cu:6-15.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .base import FEED_FORWARDS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import MATRIX, SwiGLUSpec, TensorSpec


class SwiGLU(Part):
    capture_safe = True
    def __init__(self, spec: SwiGLUSpec):
        self.spec = spec
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        return {
            s.gate: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
            s.up: TensorSpec((s.intermediate_size, s.hidden_size), MATRIX),
            s.down: TensorSpec((s.hidden_size, s.intermediate_size), MATRIX),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        self.gate_up = Linear([tensors[s.gate], tensors[s.up]], runtime, gated=True)
        self.down = Linear([tensors[s.down]], runtime)

    takes_pending_norm = True     # the gated product applies the norm of its input itself when a step is small

    def forward(self, ctx, x, residual: torch.Tensor, then_norm=None) -> bool:
        """Adds the feed-forward's output into ``residual``; returns whether ``then_norm`` was fused.
        ``x``: the normed stream, or a :class:`PendingNorm` of it."""
        from ..kernels import ops
        if isinstance(x, PendingNorm):
            T = residual.shape[0]
            if (self.runtime.fast and x.fusable and residual.dtype == torch.float32
                    and self.gate_up.can_few(T, ops.SWIGLU) and self.down.can_few(T, ops.ACCUMULATE)):
                h = ctx.buffer("ffn_hidden", (T, self.spec.intermediate_size), torch.bfloat16)
                with ops.section("ffn.gate_up"):
                    self.gate_up.few(x.source, h, ops.SWIGLU, norm=x.norm)
                with ops.section("ffn.down"):
                    self.down.few(h, residual, ops.ACCUMULATE)
                return False
            x = x.tensor()
        h = ctx.buffer("ffn_hidden", (x.shape[0], self.spec.intermediate_size), self.runtime.act_dtype)
        with ops.section("ffn.gate_up"):
            self.gate_up.swiglu(x, h, ctx)
        with ops.section("ffn.down"):
            return self.down.accumulate(h, residual, ctx, then_norm)


FEED_FORWARDS.register("swiglu", SwiGLU)
