"""A batch that decodes on the device: greedy feedback without the host in the loop.

The reference captures its one-token forward pass in a CUDA graph and replays it per
token, with position and length read from device memory (java21
inference/CudaForwardPass.java:1760-1812); its device argmax exists but the loop samples
on the host (:1353-1371). Here the captured step is the engine's own model walk for the
batch, followed by the device sampler (greedy) and a kernel that feeds the chosen tokens
back and advances every sequence, so that steps follow one another on the stream.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..cache.pages import PAGE_SIZE
from ..kernels import ops
from ..sampling.sampler import PARAMS_DTYPE
from .step import SequenceStep, StepContext


class DecodeSession:
    def __init__(self, engine, prompts: Sequence[Sequence[int]], *, reserve: int, use_graph: bool = True):
        """Prefill ``prompts`` together, then be ready to decode up to a length of ``reserve``."""
        self.engine = engine
        self.batch = B = len(prompts)
        self.slots: List[int] = [engine.acquire() for _ in prompts]
        self.closed = False
        try:
            logits = engine.step([(s, list(p)) for s, p in zip(self.slots, prompts)],
                                 [[len(p) - 1] for p in prompts])
            dev = engine.runtime.device
            V = engine.vocab_size
            # greedy parameters, one record per sequence, constant over the session
            params = np.zeros(B, dtype=PARAMS_DTYPE)
            for i in range(B):
                params[i] = (0.0, 0, 1.0, 0.0, -1.0, 0.0, 0, 0, i)
            self._params = torch.from_numpy(params.view(np.uint8).copy()).to(dev)
            self._edit_i = torch.zeros(1, dtype=torch.int32, device=dev)
            self._edit_f = torch.ones(1, dtype=torch.float32, device=dev)
            self._work = torch.empty((B, V), dtype=torch.float32, device=dev)
            self.sampled = torch.empty(B, dtype=torch.int32, device=dev)
            self._prob = torch.empty(B, dtype=torch.float32, device=dev)
            self._sample(logits)
            lengths = [engine.length(s) for s in self.slots]
            engine.cache.reserve_up_to(self.slots, [max(reserve, n + 1) for n in lengths])
            seqs = [SequenceStep(s, i, 1, n) for i, (s, n) in enumerate(zip(self.slots, lengths))]
            self.ctx = StepContext(engine.workspace, seqs, [0] * B, engine.cache.page_tables(self.slots),
                                   list(range(B)), meta_name="decode_meta")
            self.ctx.tokens.copy_(self.sampled)
            tables = engine.cache.page_tables(self.slots)
            self.capacity = min(len(t) for t in tables[0]) * PAGE_SIZE if tables else reserve
            self.steps_done = 0
            self.first_length = lengths
            self._graph = None
            self._use_graph = use_graph and engine.runtime.fast
            self.launches_per_step = 0
            self.generated: List[torch.Tensor] = [self.sampled.clone()]
        except BaseException:
            self.close()
            raise

    def _sample(self, logits: torch.Tensor) -> None:
        ops.argmax(logits, self._work.view(-1), self.sampled)

    def _one_step(self) -> None:
        eng, ctx = self.engine, self.ctx
        logits = eng.workspace.get("logits", (self.batch, eng.vocab_size), torch.float32)
        eng.model.forward(ctx, eng.cache, ctx.rows, logits)
        self._sample(logits)
        ops.advance(ctx.tokens, ctx.positions, ctx.kv_len, self.sampled)

    def run(self, steps: int, keep_tokens: bool = False) -> None:
        """``steps`` decode steps, one after another on the stream."""
        if max(self.first_length) + 1 + self.steps_done + steps > self.capacity:
            raise ValueError(f"the session reserved room for a length of {self.capacity} only")
        for _ in range(steps):
            if self._use_graph and self._graph is None and self.steps_done >= 1:
                version = self.engine.workspace.version
                before = ops.launch_count()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._one_step()
                self.launches_per_step = ops.launch_count() - before
                assert version == self.engine.workspace.version, "a buffer moved during capture"
                self._graph = graph
                # the capture itself ran nothing: replay below performs the step
            if self._graph is not None:
                self._graph.replay()
            else:
                before = ops.launch_count()
                self._one_step()
                self.launches_per_step = ops.launch_count() - before
            self.steps_done += 1
            self.engine.cache.commit(self.slots, [1] * self.batch)
            if keep_tokens:
                self.generated.append(self.sampled.clone())

    def tokens(self) -> List[List[int]]:
        """Generated tokens per sequence (the first one comes from the prompt's logits)."""
        rows = torch.stack(self.generated).cpu().tolist()
        return [list(col) for col in zip(*rows)]

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        self._graph = None
        for s in self.slots:
            try:
                self.engine.release(s)
            except Exception:
                pass
