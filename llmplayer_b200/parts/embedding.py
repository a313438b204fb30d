"""Token embedding and the head that turns the last hidden states into logits.

Reference: the embedding row is taken unscaled (inference/InferenceEngine.java:199-208);
final norm and head :225-262; a tied head re-uses the embedding table
(model/ModelLoader.java:207-214). Only the rows whose logits are wanted are normed
and projected, as the reference's prefill helper skips the head for all but the last
token (inference/InferenceEngine.java:374-381).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import NORMS, Part, Runtime
from .linear import Linear
from .specs import MATRIX, EmbeddingSpec, HeadSpec, TensorSpec


class Embedding(Part):
    capture_safe = True
    def __init__(self, spec: EmbeddingSpec):
        self.spec = spec
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.spec.weight: TensorSpec((self.spec.vocab_size, self.spec.hidden_size), MATRIX)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime, shared: Optional[torch.Tensor] = None):
        super().load(tensors, runtime)
        self.table = shared if shared is not None else runtime.matrix(tensors[self.spec.weight])

    def forward(self, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        with ops.section("embedding"):
            return ops.embed(self.table, tokens, out)

class LinearHead(Part):
    def __init__(self, spec: HeadSpec):
        self.spec = spec
        self.norm = NORMS.build(spec.norm)
        self.proj: Optional[Linear] = None

    @property
    def capture_safe(self) -> bool:
        return bool(getattr(self.norm, "capture_safe", False))

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out = dict(self.norm.tensor_specs())
        out[self.spec.weight] = TensorSpec((self.spec.vocab_size, self.spec.hidden_size), MATRIX)
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        self.norm.load(tensors, runtime)
        self.proj = Linear([tensors[self.spec.weight]], runtime)

    def forward(self, ctx, residual: torch.Tensor, rows: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """logits[i] = head(norm(residual[rows[i]])), float32."""
        if (self.runtime.fast and ctx.wanted_rows == list(range(residual.shape[0])) and residual.dtype == torch.float32
                and getattr(self.norm, "fusable_rms", False) and self.proj.can_few(residual.shape[0], ops.STORE)):
            # every token's logits are wanted and the tokens are few (a decode step): the product applies the
            # norm to the stream itself on the way in
            with ops.section("head.proj"):
                self.proj.few(residual, logits, ops.STORE, norm=self.norm)
            return logits
        h = ctx.buffer("head_in", (rows.numel(), self.spec.hidden_size), self.runtime.act_dtype)
        with ops.section("head.norm"):
            self.norm.apply(residual, h, rows=rows)
        with ops.section("head.proj"):
            return self.proj.store(h, logits, ctx)
