"""One layer: the arrangement of its norms, its mixer and its feed-forward.

``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream
x in float32 (inference/TransformerBlock.java:73-78, :109, :116-122, :149).
"""
from __future__ import annotations

import inspect
from typing import Dict, Mapping

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, FollowingNorm, Part, PendingNorm, Runtime
from .specs import BlockSpec, TensorSpec


class PreNormBlock(Part):
    def __init__(self, spec: BlockSpec):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.ffn_norm = NORMS.build(spec.ffn_norm)
        self.ffn = FEED_FORWARDS.build(spec.ffn)
        # parts may offer to write the norm that follows them (a `then_norm` argument of forward)
        self._mixer_fuses = "then_norm" in inspect.signature(self.mixer.forward).parameters
        self._ffn_fuses = "then_norm" in inspect.signature(self.ffn.forward).parameters

    def children(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    @property
    def capture_safe(self) -> bool:
        return all(bool(getattr(part, "capture_safe", False)) for part in self.children())

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

    def forward(self, ctx, cache, residual: torch.Tensor, normed_ready: bool = False, next_block=None) -> bool:
        """Run the layer on the residual stream in place.

        ``normed_ready``: the previous block already left ``norm(residual)`` of this block's first
        norm in the shared "normed" buffer. ``next_block``: the block that runs next, so that this
        block's last product can write that block's first norm on the way. Returns whether it did.
        """
        act = self.runtime.act_dtype
        tokens = residual.shape[0]
        h = ctx.buffer("normed", tuple(residual.shape), act)

        def pending(norm, consumer):
            def run():
                self._norm(ctx, norm, consumer, residual, h)
                return h
            return PendingNorm(residual, norm, run)

        # a part that takes a pending norm gets (stream, norm) and may apply the norm in its first product
        mixer_pends = bool(getattr(self.mixer, "takes_pending_norm", False))
        ffn_pends = bool(getattr(self.ffn, "takes_pending_norm", False))
        if normed_ready:
            mixer_in = h
        elif mixer_pends:
            mixer_in = pending(self.mixer_norm, self.mixer)
        else:
            self._norm(ctx, self.mixer_norm, self.mixer, residual, h)
            mixer_in = h
        fused = False
        if self._mixer_fuses and not ffn_pends:
            follow = FollowingNorm(self.ffn_norm, h, self._clear_for(ctx, self.ffn, tokens))
            fused = bool(self.mixer.forward(ctx, cache, mixer_in, residual, then_norm=follow))
            if fused and follow.clear is not None:
                ctx.note_cleared()
        else:
            self.mixer.forward(ctx, cache, mixer_in, residual)
        if fused:
            ffn_in = h
        elif ffn_pends:
            ffn_in = pending(self.ffn_norm, self.ffn)
        else:
            self._norm(ctx, self.ffn_norm, self.ffn, residual, h)
            ffn_in = h
        nxt = getattr(next_block, "mixer_norm", None)
        next_pends = bool(getattr(getattr(next_block, "mixer", None), "takes_pending_norm", False))
        if self._ffn_fuses and nxt is not None and getattr(next_block, "kind_prenorm", False) and not next_pends:
            follow = FollowingNorm(nxt, h, self._clear_for(ctx, next_block.mixer, tokens))
            done = bool(self.ffn.forward(ctx, ffn_in, residual, then_norm=follow))
            if done and follow.clear is not None:
                ctx.note_cleared()
            return done
        self.ffn.forward(ctx, ffn_in, residual)
        return False

    kind_prenorm = True

    @staticmethod
    def _clear_for(ctx, consumer, tokens):
        ask = getattr(consumer, "buffer_to_clear", None)
        return ask(ctx, tokens) if ask is not None else None

    @staticmethod
    def _norm(ctx, norm, consumer, residual, h) -> None:
        """Norm the residual stream for ``consumer``; if the consumer's first product wants a
        zeroed buffer (``buffer_to_clear(ctx, tokens)``), the norm clears it on the side."""
        clear = PreNormBlock._clear_for(ctx, consumer, residual.shape[0])
        with ops.section("norm"):
            if clear is not None:
                norm.apply(residual, h, clear=clear)
                ctx.note_cleared()
            else:
                norm.apply(residual, h)


BLOCKS.register("prenorm", PreNormBlock)
