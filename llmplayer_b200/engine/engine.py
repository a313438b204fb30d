"""The engine: a loaded model, its cache, and the one step function everything uses.

Reference: api/LLMEngine.java:233-350 (``load(path, contextLength)``), :941-1033
(``forwardSingleToken`` / ``forwardBatch``: logits for given tokens), and
inference/InferenceEngine.java:180-191 (one token of one sequence per call). Here
one call runs the new tokens of a whole batch: all prompts of a batch in one step,
then one token for each sequence, always from the cache that earlier steps left.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..cache.pages import PAGE_SIZE
from ..cache.sequence_cache import SequenceCache
from ..config.registry import ArchitectureConfig, load_config
from ..errors import LLMPlayerError, RequestError
from ..kernels import ops
from ..parts.base import Runtime
from ..weights.loader import load_tensors
from .model import Model
from .step import SequenceStep, StepContext, Workspace


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class Engine:
    def __init__(self, config: ArchitectureConfig, model: Model, runtime: Runtime, *, max_tokens: int,
                 max_slots: Optional[int] = None, context_length: Optional[int] = None):
        self.config = config
        self.model = model
        self.runtime = runtime
        self.vocab_size = model.layout.head.vocab_size
        self.context_length = context_length if context_length is not None else config.max_positions()
        self.cache = SequenceCache(model.cache_requests(), max_tokens=max_tokens, max_slots=max_slots,
                                   kv_dtype=runtime.kv_dtype, device=runtime.device)
        self.workspace = Workspace(runtime.device)
        self._sampler = None
        self.last_generation_stats = None
        self.last_step_h2d_bytes = 0
        self.use_graphs = True
        self._graphs = {}
        self._last_ctx: Optional[StepContext] = None
        self._prepared = None          # (context, page tables): the next decode step's pages, reserved ahead

    # ------------------------------------------------------------------ construction
    @classmethod
    def load(cls, model_dir: str, *, dtype: str = "bfloat16", context_length: Optional[int] = None,
             max_batch: int = 1, max_tokens: Optional[int] = None, max_slots: Optional[int] = None,
             device: str = "cuda:0", kernels: str = "fast") -> "Engine":
        """Load ``config.json`` and ``model.safetensors`` from ``model_dir``.

        ``context_length`` caps each sequence (default and upper bound: the model's
        ``max_position_embeddings``, as api/LLMEngine.java:348 takes the smaller of
        the two); the cache holds ``max_tokens`` positions in all, by default
        ``max_batch`` sequences of that length.
        """
        ops.require_gpu()
        config = load_config(model_dir)
        dev = torch.device(device)
        torch.cuda.set_device(dev)
        runtime = Runtime(device=dev, dtype=dtype, kernels=kernels)
        model = Model(config.layout())
        tensors = load_tensors(model_dir, model.tensor_specs())
        model.load(tensors, runtime)
        del tensors
        limit = config.max_positions()
        ctx_len = limit if context_length is None else min(int(context_length), limit)
        if max_tokens is None:
            max_tokens = max(1, max_batch) * _round_up(ctx_len, PAGE_SIZE)
        return cls(config, model, runtime, max_tokens=max_tokens, max_slots=max_slots, context_length=ctx_len)

    def close(self) -> None:
        self.cache = None
        self.model = None
        self.workspace = None

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        """A slot for a new sequence (``createState`` in inference/InferenceEngine.java:172-174)."""
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------------ the step
    def plan(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Sequence[Sequence[int]]) -> StepContext:
        """Check a step, reserve its pages and describe it to the device."""
        if len(entries) != len(want):
            raise RequestError(f"{len(entries)} entries but {len(want)} lists of wanted places")
        if not entries:
            raise RequestError("a step needs at least one sequence")
        sequences: List[SequenceStep] = []
        tokens: List[int] = []
        rows: List[int] = []
        for (slot, toks), places in zip(entries, want):
            toks = [int(t) for t in toks]
            if not toks:
                raise RequestError(f"slot {slot}: a step must bring at least one token")
            bad = [t for t in toks if not 0 <= t < self.vocab_size]
            if bad:
                raise RequestError(f"slot {slot}: token id {bad[0]} lies outside the vocabulary of {self.vocab_size}")
            have = self.cache.length(slot)
            if have + len(toks) > self.context_length:
                raise RequestError(
                    f"slot {slot}: {have} cached + {len(toks)} new tokens exceed the context length "
                    f"of {self.context_length}")
            for p in places:
                if not 0 <= int(p) < len(toks):
                    raise RequestError(f"slot {slot}: wanted place {p} is not among its {len(toks)} new tokens")
                rows.append(len(tokens) + int(p))
            sequences.append(SequenceStep(slot, len(tokens), len(toks), have))
            tokens.extend(toks)
        slots = [s.slot for s in sequences]
        counts = [s.num_new for s in sequences]
        self.cache.reserve(slots, counts)
        tables = self.cache.page_tables(slots)
        width = 1
        if all(n == 1 for n in counts):
            # steps of one token each are replayed from captured graphs: keep the shape of the
            # page tables stable while sequences grow (padding entries are never read)
            longest = max((len(t) for group in tables for t in group), default=1)
            width = -(-longest // 8) * 8
        return StepContext(self.workspace, sequences, tokens, tables, rows, min_table_width=width)

    def run(self, ctx: StepContext) -> torch.Tensor:
        """Run a planned step; returns float32 logits [wanted, vocab] (valid until the next step)."""
        logits = self.workspace.get("logits", (ctx.num_wanted, self.vocab_size), torch.float32)
        self.last_step_h2d_bytes = ctx.h2d_bytes
        try:
            if self.use_graphs and self.runtime.fast and ctx.all_single:
                self._run_captured(ctx, logits)
            else:
                self.model.forward(ctx, self.cache, ctx.rows, logits)
        except BaseException:
            # a step that broke off may have left partial sums behind in buffers that are zero between uses
            self._last_ctx = None
            try:
                self.workspace.restore_zeroes()
            except Exception:
                pass
            raise
        self.cache.commit(ctx.slot_list, ctx.new_counts)
        return logits

    def _run_captured(self, ctx: StepContext, logits: torch.Tensor) -> None:
        """A step of one token per sequence, through a CUDA graph of the model walk for its shape
        (batch, page-table widths, wanted rows). The first step of a shape runs directly, the
        second is captured, later ones are replayed; the step's integers were copied to the
        device beforehand, and the graph reads them there (the reference replays its captured
        forward pass the same way: java21 inference/CudaForwardPass.java:1760-1812)."""
        key = ctx.graph_key
        if key is None:
            key = ctx.graph_key = (ctx.num_sequences, tuple(t.shape[1] for t in ctx.page_tables), ctx.num_wanted,
                                   ctx.meta.data_ptr())
        entry = self._graphs.get(key)
        if entry is not None and entry[1] != self.workspace.version:
            entry = None                                  # a buffer moved since the capture
        if entry is None:
            self.model.forward(ctx, self.cache, ctx.rows, logits)
            self._graphs[key] = (None, self.workspace.version)
            return
        graph = entry[0]
        if graph is None:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.model.forward(ctx, self.cache, ctx.rows, logits)
            if entry[1] != self.workspace.version:        # should not happen: the first run sized everything
                self._graphs.pop(key, None)
                self.model.forward(ctx, self.cache, ctx.rows, logits)
                return
            if len(self._graphs) > 64:
                self._graphs.clear()
            self._graphs[key] = (graph, entry[1])
        graph.replay()

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Sequence[Sequence[int]]) -> torch.Tensor:
        """Run the given new tokens of each slot, as one batch, from the cache.

        ``entries``: ``(slot, new token ids)`` per sequence; ``want[i]``: the places
        among sequence i's new tokens whose logits are returned, in order.
        """
        ctx = self._continue(entries, want)
        if ctx is None:
            ctx = self.plan(entries, want)
        self._last_ctx = ctx if ctx.all_single else None
        return self.run(ctx)

    def _continue(self, entries, want) -> Optional[StepContext]:
        """The previous step's description moved on by one token, when this step brings one token
        for each of the same sequences and wants the same rows (the usual decode step); else None."""
        last = self._last_ctx
        if last is None or len(entries) != last.num_sequences or not last.continues_all:
            return None
        tokens: List[int] = []
        vocab, limit, cache = self.vocab_size, self.context_length, self.cache
        for (slot, toks), places, held, pos in zip(entries, want, last.slot_list, last.first_positions):
            if slot != held or len(toks) != 1 or len(places) != 1 or places[0] != 0:
                return None
            tok = int(toks[0])
            if not 0 <= tok < vocab:
                return None                     # the full check in plan() raises the error
            # the slot is still held, has room, and nothing else ran on it meanwhile
            if not cache.slots.is_held(slot) or cache.length(slot) != pos + 1 or pos + 2 > limit:
                return None
            tokens.append(tok)
        slots = last.slot_list
        prepared, self._prepared = self._prepared, None
        if prepared is not None and prepared[0] is last:
            tables = prepared[1]                # reserved while the device was still busy with the last step
        else:
            self.cache.reserve(slots, [1] * len(slots))
            tables = self.cache.page_tables(slots)
        if not last.advance(tokens, tables):
            return None
        return last

    def _prepare_continue(self) -> None:
        """Called while the device works on the step just launched: reserve the pages of the next
        one-token step of the same sequences, which needs no token. Harmless if that step never comes."""
        self._prepared = None
        last = self._last_ctx
        if last is None:
            return
        slots = last.slot_list
        for slot, pos in zip(slots, last.first_positions):
            if not self.cache.slots.is_held(slot) or self.cache.length(slot) != pos + 1 or pos + 2 > self.context_length:
                return
        try:
            self.cache.reserve(slots, [1] * len(slots))
        except LLMPlayerError:
            return                              # the step itself will report it
        self._prepared = (last, self.cache.page_tables(slots))

    # ------------------------------------------------------------------ generation
    def sample(self, logits: torch.Tensor, rows: Sequence[int], samplers) -> List[int]:
        """One token for each sampler from row ``rows[i]`` of ``logits``, drawn on the device."""
        if self._sampler is None:
            from ..sampling.sampler import BatchSampler
            self._sampler = BatchSampler(self.vocab_size, self.runtime.device)
        return self._sampler.sample(logits, rows, samplers, while_waiting=self._prepare_continue)

    def fits(self, token_counts: Sequence[int]) -> bool:
        """Whether sequences of these final lengths can be held at once, beside what is held now."""
        need = sum(-(-int(n) // PAGE_SIZE) for n in token_counts)
        return (len(token_counts) <= self.cache.slots.num_free
                and all(need <= free for free in self.cache.free_pages()))

    def generate(self, prompts, sampler_config=None, *, max_tokens: int = 256, stop_token_ids=None,
                 on_token=None, max_batch: Optional[int] = None):
        """Generate for a batch of prompts (lists of token ids) or of
        :class:`GenerationRequest`; returns one :class:`GenerationResponse` each, in order.

        Mirrors ``engine.generate(request[, callback])`` (api/LLMEngine.java:356-468):
        a prompt, a token budget, sampler options; ``on_token(request_index, token_id)``
        may return False to stop that request. ``stats`` of the last call are kept in
        ``last_generation_stats``.
        """
        from ..sampling.params import SamplerConfig
        from .generate import GenerationLoop, GenerationRequest
        requests = []
        for p in prompts:
            if isinstance(p, GenerationRequest):
                requests.append(p)
            else:
                requests.append(GenerationRequest(
                    prompt_ids=list(p), max_tokens=max_tokens,
                    sampler_config=sampler_config if sampler_config is not None else SamplerConfig(),
                    stop_token_ids=stop_token_ids))
        loop = GenerationLoop(self, max_batch=max_batch or self.cache.max_slots,
                              context_length=self.context_length,
                              default_stop_ids=self.config.stop_token_ids())
        out = loop.run(requests, on_token=on_token)
        self.last_generation_stats = loop.stats
        self.check()
        return out

    def check(self) -> None:
        """Raise if a kernel with bounded waits reported that one of them ran out since the last check
        (reads one word back from the device, which synchronises)."""
        try:
            ops.check_kernel_status()
        except BaseException:
            self._last_ctx = None
            self.workspace.restore_zeroes()
            raise

    # ------------------------------------------------------------------ reporting
    def info(self) -> str:
        lines = [self.config.describe() if hasattr(self.config, "describe") else repr(self.config)]
        lines.append(f"dtype: {self.runtime.dtype} ({self.runtime.kernels} kernels), device {self.runtime.device}")
        lines.append(f"context length: {self.context_length}; cache: {self.cache.num_pages} pages of {PAGE_SIZE} "
                     f"positions, {self.cache.max_slots} slots, {self.cache.memory_bytes() / 2**20:.1f} MiB")
        return "\n".join(lines)
