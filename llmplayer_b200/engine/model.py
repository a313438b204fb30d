"""A model: the parts of a layout, built, loaded and run in the schedule's order.

Reference: inference/InferenceEngine.java:53-101 builds the parts once;
:193-270 runs embedding, every layer, final norm and head for one token. Here
the same walk takes all tokens of a step at once, and the order of layers is the
layout's list of runs (a layer may run twice, or attend over an earlier run's cache).
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Mapping, Optional

import torch

from ..errors import ConfigError
from ..parts import BLOCKS
from ..parts.base import Runtime
from ..parts.embedding import Embedding, LinearHead
from ..parts.specs import ModelLayout, TensorSpec


class Model:
    def __init__(self, layout: ModelLayout):
        self.layout = layout
        self.embedding = Embedding(layout.embedding)
        self.blocks = [BLOCKS.build(spec) for spec in layout.layers]
        self.head = LinearHead(layout.head)
        self.runs = layout.run_order()
        for i, run in enumerate(self.runs):
            if not 0 <= run.layer < len(self.blocks):
                raise ConfigError(f"run {i} names layer {run.layer}, the model has {len(self.blocks)}")
            if run.reads_cache_of is not None and not 0 <= run.reads_cache_of < i:
                raise ConfigError(f"run {i} reads the cache of run {run.reads_cache_of}, which does not precede it")
        self.runtime: Optional[Runtime] = None
        # blocks whose forward takes (normed_ready, next_block) can hand a fused norm to the next block
        self._chains = ["next_block" in inspect.signature(b.forward).parameters for b in self.blocks]

    @property
    def capture_safe(self) -> bool:
        """Whether a captured graph of a one-token step may be replayed for other sequences: every part
        must read the step from device tensors only (``Part.capture_safe``)."""
        return all(bool(getattr(p, "capture_safe", False)) for p in [self.embedding, self.head] + self.blocks)

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Every tensor of the model folder, in a fixed order: embedding, layers, final norm, head."""
        out: Dict[str, TensorSpec] = {}
        parts = [self.embedding] + self.blocks + [self.head]
        for part in parts:
            for name, spec in part.tensor_specs().items():
                if name in out and out[name] != spec:
                    raise ConfigError(f"tensor {name!r} is asked for with shapes {out[name].shape} and {spec.shape}")
                out[name] = spec
        return out

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.embedding.load(tensors, runtime)
        for block in self.blocks:
            block.load(tensors, runtime)
        self.head.load(tensors, runtime)
        runtime.forget_uploads()

    # ------------------------------------------------------------------ cache
    def cache_requests(self) -> List[object]:
        """What each run keeps per sequence; a run that reads another's cache keeps nothing."""
        return [None if run.reads_cache_of is not None else self.blocks[run.layer].cache_request()
                for run in self.runs]

    def cache_owner(self, run_index: int) -> int:
        ref = self.runs[run_index].reads_cache_of
        return run_index if ref is None else ref

    # ------------------------------------------------------------------ a step
    def forward(self, ctx, cache, rows: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """Run the step's tokens through every run and fill ``logits[i]`` for token ``rows[i]``."""
        d = self.layout.embedding.hidden_size
        x = ctx.buffer("residual", (ctx.num_tokens, d), torch.float32)
        self.embedding.forward(ctx.tokens, x)
        ready = False        # whether the previous block already normed the stream for this one
        for i, run in enumerate(self.runs):
            block = self.blocks[run.layer]
            following = self.blocks[self.runs[i + 1].layer] if i + 1 < len(self.runs) else None
            if self._chains[run.layer]:
                ready = bool(block.forward(ctx, cache.view(self.cache_owner(i)), x, normed_ready=ready,
                                           next_block=following))
            else:
                block.forward(ctx, cache.view(self.cache_owner(i)), x)
                ready = False
        if rows.numel():
            self.head.forward(ctx, x, rows, logits)
        return logits


def expected_tensors(layout: ModelLayout) -> Dict[str, TensorSpec]:
    return Model(layout).tensor_specs()
