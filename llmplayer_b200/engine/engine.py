"""The engine: a loaded model, its cache, and the one step function everything uses.

Reference: api/LLMEngine.java:233-350 (``load(path, contextLength)``), :941-1033
(``forwardSingleToken`` / ``forwardBatch``: logits for given tokens), and
inference/InferenceEngine.java:180-191 (one token of one sequence per call). Here
one call runs the new tokens of a whole batch: all prompts of a batch in one step,
then one token for each sequence, always from the cache that earlier steps left.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.pages import PAGE_SIZE
from ..cache.sequence_cache import SequenceCache
from ..config.registry import ArchitectureConfig, load_config
from ..errors import LLMPlayerError, RequestError
from ..kernels import ops
from ..parts.base import Runtime
from ..weights.loader import load_tensors
from .model import Model
from .options import EngineOptions
from .step import SequenceStep, StepContext, Workspace


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class Engine:
    def __init__(self, config: ArchitectureConfig, model: Model, runtime: Runtime, *, max_tokens: int,
                 max_slots: Optional[int] = None, context_length: Optional[int] = None,
                 options: Optional[EngineOptions] = None):
        self.config = config
        self.model = model
        self.runtime = runtime
        self.options = options if options is not None else EngineOptions(dtype=runtime.dtype, kernels=runtime.kernels)
        self.vocab_size = model.layout.head.vocab_size
        self.context_length = context_length if context_length is not None else config.max_positions()
        self.cache = SequenceCache(model.cache_requests(), max_tokens=max_tokens, max_slots=max_slots,
                                   kv_dtype=runtime.kv_dtype, device=runtime.device)
        self.workspace = Workspace(runtime.device)
        self._sampler = None
        self.last_generation_stats = None
        self.last_step_h2d_bytes = 0
        self.last_step_d2h_bytes = 0
        self.profiler: Optional[ops.StepProfiler] = ops.StepProfiler() if self.options.profile else None
        self.use_graphs = bool(self.options.graphs) and not self.options.profile
        self._graphs = {}
        self._fused = {}               # captured decode steps with upload, argmax and read-back inside
        self._last_ctx: Optional[StepContext] = None
        self._prepared = None          # (context, page tables): the next decode step's pages, reserved ahead

    # ------------------------------------------------------------------ construction
    @classmethod
    def load(cls, model_dir: str, options: Optional[EngineOptions] = None, **changes) -> "Engine":
        """Load ``config.json`` and ``model.safetensors`` from ``model_dir``.

        ``options`` (an :class:`EngineOptions`) and/or its fields as keyword arguments: ``dtype``,
        ``kernels``, ``context_length``, ``max_batch``, ``max_tokens``, ``max_slots``, ``device``,
        ``graphs``, ``profile``, kernel switches. ``context_length`` caps each sequence (default and
        upper bound: the model's ``max_position_embeddings``, as api/LLMEngine.java:348 takes the
        smaller of the two; ``beyond_model_context=True`` lifts the upper bound); the cache holds
        ``max_tokens`` positions in all, by default ``max_batch`` sequences of that length.
        """
        ops.require_gpu()
        opts = (options if options is not None else EngineOptions()).with_changes(**changes)
        if opts.kernel_settings():
            ops.configure(**opts.kernel_settings())
        config = load_config(model_dir)
        dev = torch.device(opts.device)
        torch.cuda.set_device(dev)
        runtime = Runtime(device=dev, dtype=opts.dtype, kernels=opts.kernels)
        model = Model(config.layout())
        tensors = load_tensors(model_dir, model.tensor_specs())
        model.load(tensors, runtime)
        del tensors
        limit = config.max_positions()
        if opts.context_length is None:
            ctx_len = limit
        elif opts.beyond_model_context:
            ctx_len = int(opts.context_length)
        else:
            ctx_len = min(int(opts.context_length), limit)
        max_tokens = opts.max_tokens
        if max_tokens is None:
            max_tokens = max(1, opts.max_batch) * _round_up(ctx_len, PAGE_SIZE)
        return cls(config, model, runtime, max_tokens=max_tokens, max_slots=opts.max_slots, context_length=ctx_len,
                   options=opts)

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
            # page tables stable while sequences grow (padding entries are never read). The width doubles
            # when the longest table has come within a page of it, so that a batch is captured anew a
            # handful of times in its life and not every 512 tokens.
            longest = max((len(t) for group in tables for t in group), default=1)
            width = 8
            while width < longest + 1:
                width *= 2
        return StepContext(self.workspace, sequences, tokens, tables, rows, min_table_width=width)

    def run(self, ctx: StepContext) -> torch.Tensor:
        """Run a planned step; returns float32 logits [wanted, vocab] (valid until the next step)."""
        logits = self.workspace.get("logits", (ctx.num_wanted, self.vocab_size), torch.float32)
        self.last_step_h2d_bytes = ctx.h2d_bytes
        try:
            if self.profiler is not None:
                ops.set_profiler(self.profiler)
                try:
                    self.model.forward(ctx, self.cache, ctx.rows, logits)
                    self.profiler.steps += 1
                finally:
                    ops.set_profiler(None)
            elif self.use_graphs and self.runtime.fast and ctx.all_single and self.model.capture_safe:
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

    def _continue(self, entries, want, advance: bool = True) -> Optional[StepContext]:
        """The previous step's description moved on by one token, when this step brings one token
        for each of the same sequences and wants the same rows (the usual decode step); else None.
        ``advance=False``: only say whether it applies (the context is returned as it is)."""
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
        if not advance:
            return last
        slots = last.slot_list
        prepared, self._prepared = self._prepared, None
        if prepared is not None and prepared[0] is last:
            tables = prepared[1]                # reserved while the device was still busy with the last step
        else:
            self.cache.reserve(slots, [1] * len(slots))
            tables = self.cache.page_tables(slots)
        if last.advance(tokens, tables) is None:
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
        if self.profiler is not None:
            ops.set_profiler(self.profiler)
        try:
            chosen = self._sampler.sample(logits, rows, samplers, while_waiting=self._prepare_continue)
        finally:
            ops.set_profiler(None)
        self.last_step_d2h_bytes = self._sampler.last_d2h_bytes
        self.last_step_h2d_bytes += self._sampler.last_h2d_bytes
        return chosen

    def decode_steps(self, entries: Sequence[Tuple[int, int]], samplers, *, quiet: Optional[Sequence[int]] = None,
                     stops: Optional[Sequence[Sequence[int]]] = None, max_steps: int = 256) -> List[List[int]]:
        """Decode: feed one token to each sequence (``entries``: ``(slot, token)``), sample each one's next
        token, and go on doing so while nothing has to be decided. Returns the chosen tokens of every step
        that ran (at least one step), oldest first.

        ``quiet[i]``: how many of sequence i's next chosen tokens are certain to need no decision other than
        "is it one of ``stops[i]``" (the generation loop knows: token budget, context). Given these, the steps
        run from the native host loop: one captured graph per step that holds the upload of the step's
        integers from page-locked memory, the model walk, the choice of the tokens and their read-back
        (csrc/host_loop.cu), until a step is not quiet. The choice is the argmax when every sampler is a plain
        greedy one; with temperature, top-k, top-p, min-p and a repetition penalty it is the sampling kernels,
        and the loop keeps each sequence's generator and window of recent tokens. Samplers with DRY or mirostat
        (state that follows the drawn probabilities or searches the history) run one step at a time through
        :meth:`step` and :meth:`sample`.
        """
        # samplers whose state the native loop keeps: a generator and the window of recent tokens
        native = all(s.plain_greedy or (s.config.mirostat == 0 and s.config.dry_multiplier <= 0) for s in samplers)
        if (quiet is not None and self.options.host_loop and self.use_graphs and self.runtime.fast
                and self.model.capture_safe and native):
            greedy = all(s.plain_greedy for s in samplers)
            out = self._decode_fused(entries, quiet, stops, max_steps, None if greedy else list(samplers))
            if out is not None:
                return out
        logits = self.step([(slot, [tok]) for slot, tok in entries], [[0]] * len(entries))
        return [self.sample(logits, list(range(len(entries))), samplers)]

    def _decode_fused(self, entries, quiet, stops, max_steps, samplers=None) -> Optional[List[List[int]]]:
        B = len(entries)
        want = [[0]] * B
        step_entries = [(slot, [tok]) for slot, tok in entries]
        last = self._continue(step_entries, want, advance=False)     # None: the first step after the prompts
        slots = [slot for slot, _ in entries]
        try:
            lengths = [self.cache.length(slot) for slot in slots]
        except LLMPlayerError:
            return None                                   # the plain way reports it
        # how many steps at most: while all stay quiet, within the context, and within the pages that can be had
        room = min(self.context_length - n for n in lengths)
        if room < 1 or len(set(slots)) != B:
            return None
        steps = max(1, min(int(max_steps), min(int(q) for q in quiet) + 1, room))
        self._prepared = None
        while True:
            try:
                self.cache.reserve(slots, [steps] * B)
                break
            except LLMPlayerError:
                if steps == 1:
                    return None                           # the plain way reports it
                steps = max(1, steps // 2)
        tables = self.cache.page_tables(slots)
        moved = None if last is None else last.advance([tok for _, tok in entries], tables, upload=False)
        if moved is None:                  # no context to move on, or the tables outgrew its shape: describe the step anew
            ctx = self.plan(step_entries, want)
        else:
            ctx = last
            if moved:                                     # page tables changed: they are not part of the graph's own copy
                ctx.upload_all()
        self._last_ctx = ctx
        key = ctx.fused_key
        if key is None:
            key = ctx.fused_key = (B, tuple(t.shape[1] for t in ctx.page_tables), ctx.meta.data_ptr(), ctx.host_pointer)
        logits = self.workspace.get("logits", (B, self.vocab_size), torch.float32)
        sampled = self.workspace.get("sampled", (B,), torch.int32)
        landing, _ = self.workspace.pinned("sampled_host", B)
        draw = None
        if samplers is None:
            work = self.workspace.get("argmax_work", (64 * B,), torch.float32)
        else:
            draw = self._sampler_block(samplers, B)
            key = key + ("sampled", draw["sliced"], draw["host"].data_ptr(), draw["cap"])
        entry = self._fused.get(key)
        if entry is not None and entry["version"] != self.workspace.version:
            entry = None

        def one_step(upload: bool, captured: bool = False):
            if upload:
                ctx.upload_moving(record=not captured)
            self.model.forward(ctx, self.cache, ctx.rows, logits)
            if draw is None:
                ops.argmax(logits, work, sampled)
            else:
                d = draw
                ops.sample_fetch(d["host"], d["dev"], B, d["cap"], d["record_words"], d["field_count"])
                ops.sample(logits, d["work"], d["params"], d["edit_tok"], d["edit_sub"], d["edit_fac"], sampled,
                           d["prob"], select=d["select"])
            landing[:B].copy_(sampled, non_blocking=True)

        try:
            if entry is None and draw is not None:
                # a shape's first step with a sampler: run once for nothing (it sizes every buffer; the step's keys
                # and values are written again, the same, by the step that counts), then capture and go on below
                one_step(upload=moved is not None)
                torch.cuda.current_stream().synchronize()
                entry = self._fused[key] = {"graph": None, "version": self.workspace.version}
            if entry is None:
                # the first step of a shape runs directly (it sizes every buffer), the second is captured
                one_step(upload=moved is not None)
                torch.cuda.current_stream().synchronize()
                self._fused[key] = {"graph": None, "version": self.workspace.version}
                chosen = [landing[:B].tolist()]
            else:
                if entry["graph"] is None:
                    graph = torch.cuda.CUDAGraph()
                    before = ops.launch_count()
                    with torch.cuda.graph(graph):
                        one_step(upload=True, captured=True)
                    if entry["version"] != self.workspace.version:
                        raise LLMPlayerError("a buffer moved while a decode step was captured")
                    if len(self._fused) > 64:
                        self._fused.clear()
                    entry = self._fused[key] = {"graph": graph, "version": entry["version"],
                                                "exec": graph.raw_cuda_graph_exec(),
                                                "launches": ops.launch_count() - before}
                if draw is None:
                    chosen = self._host_loop(ctx, entry, landing, B, steps, quiet, stops)
                else:
                    chosen = self._host_loop_sampled(ctx, entry, landing, B, steps, quiet, stops, samplers, draw)
                ops.count_launches(entry["launches"] * len(chosen))
        except BaseException:
            self._last_ctx = None
            try:
                self.workspace.restore_zeroes()
            except Exception:
                pass
            raise
        k = len(chosen)
        ctx.moved_on(k - 1)
        self.cache.commit(slots, [k] * B)
        self.last_step_h2d_bytes = ctx.moving_bytes + (0 if draw is None else 4 * B * draw["record_words"])
        self.last_step_d2h_bytes = 4 * B
        return chosen

    @staticmethod
    def _stop_arrays(B, quiet, stops):
        quiet_arr = np.asarray([int(q) for q in quiet], dtype=np.int32)
        begin = np.zeros(B + 1, dtype=np.int32)
        flat: List[int] = []
        for i in range(B):
            if stops is not None:
                flat.extend(int(t) for t in stops[i])
            begin[i + 1] = len(flat)
        return quiet_arr, begin, np.asarray(flat or [0], dtype=np.int32)

    def _sampler_block(self, samplers, B) -> dict:
        """The buffers of a captured step that draws its tokens: the sampler block (one record per sequence and room
        for the logit edits of a full window of recent tokens each) in page-locked and in device memory, and the
        sampling kernels' scratch. The records' fixed fields are written here; the native loop fills in each step's
        uniform number and edits."""
        from ..sampling.sampler import PARAMS_DTYPE
        lib = ops.library("sampling")
        record = PARAMS_DTYPE.itemsize
        if record != lib.lp_sample_params_size() or record % 4:
            raise LLMPlayerError("the sampler's parameter record and the kernel's disagree")
        words = record // 4
        cap = max(s.max_recent for s in samplers)
        total = B * (words + 3 * cap)
        host, _ = self.workspace.pinned("sample_block_host", total)
        host = host[:total]
        dev = self.workspace.get("sample_block", (total,), torch.int32)
        params = np.zeros(B, dtype=PARAMS_DTYPE)
        for i, smp in enumerate(samplers):
            c = smp.config
            params[i] = (0.0 if c.is_greedy else 1.0 / np.float32(c.temperature), c.top_k, c.top_p, c.min_p,
                         -1.0, 0.0, i * cap, 0, i)
        host.numpy()[:B * words] = params.view(np.int32)
        fields = {name: PARAMS_DTYPE.fields[name][1] // 4 for name in ("uniform", "edit_begin", "edit_count")}
        capacity = ops.sample_slice_capacity(self.vocab_size)
        sliced = any(not smp.config.is_greedy and 0 < smp.config.top_k <= capacity for smp in samplers)
        head = B * words
        return {
            "host": host, "dev": dev, "cap": cap, "record_words": words, "field_count": fields["edit_count"],
            "field_uniform": fields["uniform"], "field_begin": fields["edit_begin"], "sliced": sliced,
            "params": dev[:head].view(torch.uint8), "edit_tok": dev[head:head + B * cap],
            "edit_sub": dev[head + B * cap:head + 2 * B * cap].view(torch.float32),
            "edit_fac": dev[head + 2 * B * cap:head + 3 * B * cap].view(torch.float32),
            "work": self.workspace.get("sample_work", (B, self.vocab_size), torch.float32),
            "prob": self.workspace.get("sample_prob", (B,), torch.float32),
            "select": (self.workspace.get("sample_select", (B * ops.sample_select_words(),), torch.int32)
                       if sliced else None),
        }

    def _host_loop_sampled(self, ctx, entry, landing, B, steps, quiet, stops, samplers, draw) -> List[List[int]]:
        """The native loop with the samplers' state (csrc/host_loop.cu: lp_decode_loop_sampled); the samplers take
        over the generators' states and the windows of recent tokens it leaves."""
        lib = ops.library("host_loop")
        quiet_arr, begin, stop_arr = self._stop_arrays(B, quiet, stops)
        cap = draw["cap"]
        rng = np.asarray([smp.rng._state for smp in samplers], dtype=np.uint64)
        draws = np.asarray([0 if smp.config.is_greedy else 1 for smp in samplers], dtype=np.int32)
        penalty = np.asarray([float(smp.config.repetition_penalty) for smp in samplers], dtype=np.float64)
        recent = np.zeros((B, cap), dtype=np.int32)
        recent_len = np.zeros(B, dtype=np.int32)
        window = np.asarray([smp.max_recent for smp in samplers], dtype=np.int32)
        for i, smp in enumerate(samplers):
            kept = smp.recent[-smp.max_recent:]
            recent[i, :len(kept)] = kept
            recent_len[i] = len(kept)
        scratch = np.zeros(2 * B * cap, dtype=np.int32)
        out = np.empty((steps, B), dtype=np.int32)
        ran = ctypes.c_int(0)
        tokens_at, positions_at, lengths_at = ctx.moving_offsets
        code = lib.lp_decode_loop_sampled(
            entry["exec"], ops.current_stream(), ctx.host_pointer, tokens_at, positions_at, lengths_at,
            draw["host"].data_ptr(), draw["record_words"], draw["field_uniform"], draw["field_begin"],
            draw["field_count"], cap, landing.data_ptr(), B, steps, quiet_arr.ctypes.data, stop_arr.ctypes.data,
            begin.ctypes.data, rng.ctypes.data, draws.ctypes.data, penalty.ctypes.data, recent.ctypes.data,
            recent_len.ctypes.data, window.ctypes.data, scratch.ctypes.data, out.ctypes.data, ctypes.byref(ran))
        for i, smp in enumerate(samplers):                   # what ran, ran: the samplers go on from there
            smp.rng._state = int(rng[i])
            smp.recent = recent[i, :int(recent_len[i])].tolist()
        if code != 0:
            raise LLMPlayerError(lib.lp_last_error().decode("utf-8", "replace") or f"decode loop failed ({code})")
        return out[:ran.value].tolist()

    def _host_loop(self, ctx, entry, landing, B, steps, quiet, stops) -> List[List[int]]:
        lib = ops.library("host_loop")
        quiet_arr, begin, stop_arr = self._stop_arrays(B, quiet, stops)
        out = np.empty((steps, B), dtype=np.int32)
        ran = ctypes.c_int(0)
        tokens_at, positions_at, lengths_at = ctx.moving_offsets
        code = lib.lp_decode_loop(entry["exec"], ops.current_stream(), ctx.host_pointer, tokens_at, positions_at,
                                  lengths_at, landing.data_ptr(), B, steps, quiet_arr.ctypes.data, stop_arr.ctypes.data,
                                  begin.ctypes.data, out.ctypes.data, ctypes.byref(ran))
        if code != 0:
            raise LLMPlayerError(lib.lp_last_error().decode("utf-8", "replace") or f"decode loop failed ({code})")
        return out[:ran.value].tolist()

    @staticmethod
    def launch_count() -> int:
        """Kernels of this library launched so far by this process (replays of captured steps included)."""
        return ops.launch_count()

    def mark(self):
        """A timing event on the current stream (for the generation loop's device-side clock)."""
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        return event

    @staticmethod
    def elapsed_ms(start, end) -> float:
        end.synchronize()
        return float(start.elapsed_time(end))

    def fits(self, token_counts: Sequence[int]) -> bool:
        """Whether sequences of these final lengths can be held at once, beside what is held now."""
        need = sum(-(-int(n) // PAGE_SIZE) for n in token_counts)
        return (len(token_counts) <= self.cache.slots.num_free
                and all(need <= free for free in self.cache.free_pages()))

    def generate(self, prompts, sampler_config=None, *, max_tokens: int = 256, stop_token_ids=None,
                 on_token=None, max_batch: Optional[int] = None, laps=None):
        """Generate for a batch of prompts (lists of token ids) or of
        :class:`GenerationRequest`; returns one :class:`GenerationResponse` each, in order.

        Mirrors ``engine.generate(request[, callback])`` (api/LLMEngine.java:356-468):
        a prompt, a token budget, sampler options; ``on_token(request_index, token_id)``
        may return False to stop that request. ``stats`` of the last call are kept in
        ``last_generation_stats``; ``laps=(skip, every)`` times the decode steps in laps (see
        :meth:`GenerationLoop.run`).
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
        out = loop.run(requests, on_token=on_token, laps=laps)
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
    def profile_report(self, reset: bool = False) -> dict:
        """Device time per section of the model walk since the engine was loaded with ``profile=True`` (or since
        the last reset): ``{"steps", "total_ms", "sections": {name: {"ms", "calls", "ms_per_step"}}}``."""
        if self.profiler is None:
            raise RequestError("this engine was not loaded with profile=True")
        report = self.profiler.report()
        if reset:
            self.profiler.reset()
        return report

    def info(self) -> str:
        lines = [self.config.describe() if hasattr(self.config, "describe") else repr(self.config)]
        lines.append(f"dtype: {self.runtime.dtype} ({self.runtime.kernels} kernels), device {self.runtime.device}")
        lines.append(f"context length: {self.context_length}; cache: {self.cache.num_pages} pages of {PAGE_SIZE} "
                     f"positions, {self.cache.max_slots} slots, {self.cache.memory_bytes() / 2**20:.1f} MiB")
        return "\n".join(lines)
