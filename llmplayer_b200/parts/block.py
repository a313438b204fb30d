"""One layer: the arrangement of its norms, its mixer and its feed-forward.

``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream
x in float32 (inference/TransformerBlock.java:73-78, :109, :116-122, :149).
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Part, Runtime
from .specs import BlockSpec, TensorSpec


class PreNormBlock(Part):
    def __init__(self, spec: BlockSpec):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.ffn_norm = NORMS.build(spec.ffn_norm)
        self.ffn = FEED_FORWARDS.build(spec.ffn)

    def children(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.children():
            out.update(part.tensor_specs())
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        for part in self.children():
            part.load(tensors, runtime)

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, ctx, cache, residual: torch.Tensor) -> None:
        act = self.runtime.act_dtype
        h = ctx.buffer("normed", tuple(residual.shape), act)
        self._norm(ctx, self.mixer_norm, self.mixer, residual, h)
        self.mixer.forward(ctx, cache, h, residual)
        self._norm(ctx, self.ffn_norm, self.ffn, residual, h)
        self.ffn.forward(ctx, h, residual)

    @staticmethod
    def _norm(ctx, norm, consumer, residual, h) -> None:
        """Norm the residual stream for ``consumer``; if the consumer's first product wants a
        zeroed buffer (``buffer_to_clear(ctx, tokens)``), the norm clears it on the side."""
        ask = getattr(consumer, "buffer_to_clear", None)
        clear = ask(ctx, residual.shape[0]) if ask is not None else None
        if clear is not None:
            norm.apply(residual, h, clear=clear)
            ctx.note_cleared()
        else:
            norm.apply(residual, h)


BLOCKS.register("prenorm", PreNormBlock)
