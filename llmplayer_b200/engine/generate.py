"""The generation loop: batches of unequal prompts, stop tokens, sequences that end
earlier, and as many batches one after another as there are requests.

Per sequence the order of decisions is the reference's (api/LLMEngine.java:743-769):
sample from the current logits; a stop token ends the sequence and is neither
emitted nor fed back (:746-749); otherwise the token is recorded and the callback
may stop the sequence (:762-764); at position >= context - 1 the sequence ends
(:766-767); else the token is fed forward. A prompt of context - 1 tokens or more
is refused with an error response, not an exception (:396-399). Tokens per second
count generated tokens over the time since the prompt was processed (:481, :772-775).

The loop talks to a *backend* (the engine, or a scripted stand-in in tests):
``acquire()``, ``release(slot)``, ``step(entries, want) -> logits``,
``sample(logits, rows, samplers) -> tokens``, ``fits(token_counts) -> bool``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.params import SamplerConfig
from ..sampling.sampler import SequenceSampler


@dataclass
class GenerationRequest:
    """api/GenerationRequest.java:49-55, with token ids in place of the prompt text."""
    prompt_ids: Sequence[int]
    max_tokens: int = 256
    sampler_config: SamplerConfig = field(default_factory=SamplerConfig)
    stop_token_ids: Optional[Sequence[int]] = None     # None: the model configuration's end tokens


@dataclass
class GenerationResponse:
    """api/GenerationResponse.java:8-13, with token ids in place of the text."""
    token_ids: List[int]
    prompt_token_count: int
    finish_reason: str                 # stop | length | context | callback | error
    tokens_per_second: float = 0.0
    time_ms: float = 0.0
    error: Optional[str] = None

    @property
    def token_count(self) -> int:
        return len(self.token_ids)


@dataclass
class GenerationStats:
    batches: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    decode_steps: int = 0
    step_tokens: int = 0              # tokens chosen from the logits of decode steps (not of the prompts)
    decode_device_ms: float = 0.0     # the decode steps' time on the device's own clock, when the backend has one
    decode_launches: int = 0          # kernels launched for the decode steps, when the backend counts them
    laps: List[dict] = field(default_factory=list)   # see GenerationLoop.run(laps=...)

    @property
    def decode_tokens_per_second(self) -> float:
        """The reference's figure: all generated tokens over the time since the prompts' logits were there
        (api/LLMEngine.java:481, :772-775), the first token of each sequence included."""
        return self.generated_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0

    @property
    def step_tokens_per_second(self) -> float:
        """Tokens that decode steps produced over the same time: the rate of the steps themselves."""
        return self.step_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0

    @property
    def device_step_tokens_per_second(self) -> float:
        return self.step_tokens / (self.decode_device_ms / 1e3) if self.decode_device_ms > 0 else 0.0


class _Live:
    def __init__(self, index: int, request: GenerationRequest, stop_ids, slot: int):
        self.index = index
        self.request = request
        self.stop_ids = stop_ids
        self.slot = slot
        self.sampler = SequenceSampler(request.sampler_config)
        self.tokens: List[int] = []
        self.next_token: Optional[int] = None
        self.finish: Optional[str] = None


class GenerationLoop:
    def __init__(self, backend, *, max_batch: int, context_length: int, default_stop_ids: Sequence[int] = ()):
        self.backend = backend
        self.max_batch = max(1, int(max_batch))
        self.context_length = int(context_length)
        self.default_stop_ids = tuple(default_stop_ids)
        self.stats = GenerationStats()
        self._laps = None

    # ------------------------------------------------------------------ batches
    def _need(self, request: GenerationRequest) -> int:
        return min(len(request.prompt_ids) + max(0, request.max_tokens), self.context_length)

    def run(self, requests: Sequence[GenerationRequest],
            on_token: Optional[Callable[[int, int], Optional[bool]]] = None,
            laps: Optional[Sequence[int]] = None) -> List[GenerationResponse]:
        """Generate for every request; responses come in request order.

        ``laps = (skip, every)``: for measurements. After the first ``skip`` decode steps of a batch, the
        decode steps are timed in laps of ``every`` steps each; ``stats.laps`` gets one entry per full lap:
        ``{"steps", "tokens", "host_ms", "device_ms", "launches"}`` (the device's clock and the launch count
        when the backend has them)."""
        self._laps = (max(0, int(laps[0])), max(1, int(laps[1]))) if laps else None
        responses: List[Optional[GenerationResponse]] = [None] * len(requests)
        pending: List[int] = []
        for i, req in enumerate(requests):
            n = len(req.prompt_ids)
            if n == 0:
                responses[i] = GenerationResponse([], 0, "error", error="Error: empty prompt")
            elif n >= self.context_length - 1:
                responses[i] = GenerationResponse(
                    [], n, "error",
                    error=f"Error: prompt too long ({n} tokens, max {self.context_length - 1})")
            elif req.max_tokens <= 0:
                responses[i] = GenerationResponse([], n, "length")
            elif not self.backend.fits([self._need(req)]):
                responses[i] = GenerationResponse(
                    [], n, "error", error=f"Error: the cache cannot hold {self._need(req)} tokens for this request")
            else:
                pending.append(i)
        while pending:
            batch: List[int] = []
            needs: List[int] = []
            while pending and len(batch) < self.max_batch:
                need = self._need(requests[pending[0]])
                if batch and not self.backend.fits(needs + [need]):
                    break
                batch.append(pending.pop(0))
                needs.append(need)
            self._run_batch(batch, requests, responses, on_token)
        return responses  # type: ignore[return-value]

    # ------------------------------------------------------------------ one batch
    def _decide(self, s: _Live, tok: int, step_index: int, on_token) -> None:
        """What becomes of sequence ``s`` after ``tok`` was chosen for it (the reference's order of decisions)."""
        if tok in s.stop_ids:
            s.finish = "stop"
            return
        s.tokens.append(tok)
        self.stats.generated_tokens += 1
        if on_token is not None and on_token(s.index, tok) is False:
            s.finish = "callback"
            return
        position = len(s.request.prompt_ids) + step_index
        if position >= self.context_length - 1:
            s.finish = "context"
        elif len(s.tokens) >= s.request.max_tokens:
            s.finish = "length"
        else:
            s.next_token = tok

    def _quiet(self, s: _Live, step_index: int) -> int:
        """How many of the sequence's next chosen tokens can only be continued or be a stop token: neither the
        token budget nor the context ends the sequence at them."""
        by_context = self.context_length - 1 - len(s.request.prompt_ids) - step_index
        by_budget = s.request.max_tokens - len(s.tokens) - 1
        return max(0, min(by_context, by_budget))

    def _run_batch(self, batch, requests, responses, on_token) -> None:
        be = self.backend
        live: List[_Live] = []
        for i in batch:
            req = requests[i]
            stop = self.default_stop_ids if req.stop_token_ids is None else tuple(req.stop_token_ids)
            live.append(_Live(i, req, frozenset(int(t) for t in stop), be.acquire()))
        self.stats.batches += 1
        several = getattr(be, "decode_steps", None)       # a backend that can run several quiet steps per call
        mark = getattr(be, "mark", None)
        count = getattr(be, "launch_count", None)
        launched = None
        t0 = time.perf_counter()
        t_decode = None
        started = None
        try:
            logits = be.step([(s.slot, list(s.request.prompt_ids)) for s in live],
                             [[len(s.request.prompt_ids) - 1] for s in live])
            pending = [be.sample(logits, list(range(len(live))), [s.sampler for s in live])]
            # the prompt is processed once its logits are there: decode time starts here
            t_decode = time.perf_counter()
            started = mark() if mark is not None else None
            launched = count() if count is not None else None
            self.stats.prefill_ms += (t_decode - t0) * 1e3
            self.stats.prompt_tokens += sum(len(s.request.prompt_ids) for s in live)
            step_index = 0
            steps_done = 0
            boundary = None                       # the decode step count at which the current lap ends
            lap_start = None                      # (host time, device mark, launches, tokens) at its beginning
            if self._laps is not None:
                boundary = self._laps[0] if self._laps[0] > 0 else self._laps[1]
                if self._laps[0] == 0:
                    lap_start = (t_decode, started, launched, 0)
            while live:
                for n, chosen in enumerate(pending):
                    for s, tok in zip(live, chosen):
                        self._decide(s, int(tok), step_index, on_token)
                    step_index += 1
                    if n + 1 < len(pending) and any(s.finish is not None for s in live):
                        raise RuntimeError("the backend ran on past a step that ended a sequence")
                now = time.perf_counter()
                for s in live:
                    if s.finish is not None:
                        elapsed = now - t_decode
                        responses[s.index] = GenerationResponse(
                            s.tokens, len(s.request.prompt_ids), s.finish,
                            tokens_per_second=len(s.tokens) / elapsed if elapsed > 0 and s.tokens else 0.0,
                            time_ms=(now - t0) * 1e3)
                        be.release(s.slot)
                        s.slot = None
                live = [s for s in live if s.finish is None]
                if not live:
                    break
                if several is not None:
                    quiet = [0 if on_token is not None else self._quiet(s, step_index) for s in live]
                    most = 256 if boundary is None else max(1, min(256, boundary - steps_done))
                    pending = several([(s.slot, s.next_token) for s in live], [s.sampler for s in live],
                                      quiet=quiet, stops=[s.stop_ids for s in live], max_steps=most)
                else:
                    logits = be.step([(s.slot, [s.next_token]) for s in live], [[0] for _ in live])
                    pending = [be.sample(logits, list(range(len(live))), [s.sampler for s in live])]
                self.stats.decode_steps += len(pending)
                self.stats.step_tokens += len(live) * len(pending)
                steps_done += len(pending)
                if boundary is not None and steps_done >= boundary:
                    here = (time.perf_counter(), mark() if mark is not None else None,
                            count() if count is not None else None, self.stats.step_tokens)
                    if lap_start is not None and steps_done == boundary:
                        lap = {"steps": self._laps[1], "tokens": here[3] - lap_start[3],
                               "host_ms": (here[0] - lap_start[0]) * 1e3}
                        if here[1] is not None and lap_start[1] is not None:
                            lap["device_ms"] = be.elapsed_ms(lap_start[1], here[1])
                        if here[2] is not None and lap_start[2] is not None:
                            lap["launches"] = here[2] - lap_start[2]
                        self.stats.laps.append(lap)
                    lap_start = here
                    boundary = steps_done + self._laps[1]
        finally:
            if t_decode is not None:
                self.stats.decode_ms += (time.perf_counter() - t_decode) * 1e3
                if launched is not None:
                    self.stats.decode_launches += count() - launched
                if started is not None:
                    try:
                        self.stats.decode_device_ms += be.elapsed_ms(started, mark())
                    except Exception:
                        pass
            for s in live:
                if s.slot is not None:
                    be.release(s.slot)
                    s.slot = None
