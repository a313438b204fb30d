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

    @property
    def decode_tokens_per_second(self) -> float:
        return self.generated_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0


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

    # ------------------------------------------------------------------ batches
    def _need(self, request: GenerationRequest) -> int:
        return min(len(request.prompt_ids) + max(0, request.max_tokens), self.context_length)

    def run(self, requests: Sequence[GenerationRequest],
            on_token: Optional[Callable[[int, int], Optional[bool]]] = None) -> List[GenerationResponse]:
        """Generate for every request; responses come in request order."""
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
    def _run_batch(self, batch, requests, responses, on_token) -> None:
        be = self.backend
        live: List[_Live] = []
        for i in batch:
            req = requests[i]
            stop = self.default_stop_ids if req.stop_token_ids is None else tuple(req.stop_token_ids)
            live.append(_Live(i, req, frozenset(int(t) for t in stop), be.acquire()))
        self.stats.batches += 1
        t0 = time.perf_counter()
        try:
            logits = be.step([(s.slot, list(s.request.prompt_ids)) for s in live],
                             [[len(s.request.prompt_ids) - 1] for s in live])
            step_index = 0
            first = True
            t_decode = None
            while live:
                chosen = be.sample(logits, list(range(len(live))), [s.sampler for s in live])
                if first:
                    # the prompt is processed once its logits are there: decode time starts here
                    t_decode = time.perf_counter()
                    self.stats.prefill_ms += (t_decode - t0) * 1e3
                    self.stats.prompt_tokens += sum(len(s.request.prompt_ids) for s in live)
                    first = False
                for s, tok in zip(live, chosen):
                    tok = int(tok)
                    if tok in s.stop_ids:
                        s.finish = "stop"
                        continue
                    s.tokens.append(tok)
                    self.stats.generated_tokens += 1
                    if on_token is not None and on_token(s.index, tok) is False:
                        s.finish = "callback"
                        continue
                    position = len(s.request.prompt_ids) + step_index
                    if position >= self.context_length - 1:
                        s.finish = "context"
                    elif len(s.tokens) >= s.request.max_tokens:
                        s.finish = "length"
                    else:
                        s.next_token = tok
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
                logits = be.step([(s.slot, [s.next_token]) for s in live], [[0] for _ in live])
                self.stats.decode_steps += 1
                step_index += 1
            if t_decode is not None:
                self.stats.decode_ms += (time.perf_counter() - t_decode) * 1e3
        finally:
            for s in live:
                if s.slot is not None:
                    be.release(s.slot)
                    s.slot = None
