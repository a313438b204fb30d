"""The generation loop's decisions, with a scripted backend in place of the engine."""
import pytest

from llmplayer_b200.engine.generate import GenerationLoop, GenerationRequest
from llmplayer_b200.sampling import SamplerConfig

STOP = 99


class ScriptedBackend:
    """Each sequence emits its script, token after token; slots come from a small pool."""

    def __init__(self, scripts, slots=8, capacity=10 ** 9):
        self.scripts = scripts            # prompt tuple -> list of tokens to emit
        self.free = list(range(slots))
        self.capacity = capacity
        self.held = {}                    # slot -> [prompt, tokens fed]
        self.steps = []                   # (kind, [slots])
        self.released = []

    def acquire(self):
        slot = self.free.pop(0)
        self.held[slot] = None
        return slot

    def release(self, slot):
        assert slot in self.held, "released a slot that is not held"
        del self.held[slot]
        self.released.append(slot)
        self.free.append(slot)

    def fits(self, counts):
        return len(counts) <= len(self.free) and sum(counts) <= self.capacity

    def step(self, entries, want):
        kind = "decode" if all(len(t) == 1 and self.held[s] is not None for s, t in entries) else "prefill"
        out = []
        for (slot, toks), w in zip(entries, want):
            if self.held[slot] is None:
                self.held[slot] = [tuple(toks), 0]
                assert w == [len(toks) - 1]
            else:
                prompt, fed = self.held[slot]
                assert toks == [self.scripts[prompt][fed]], "the sampled token must be fed back"
                self.held[slot][1] += 1
                assert w == [0]
            prompt, fed = self.held[slot]
            out.append(self.scripts[prompt][fed] if fed < len(self.scripts[prompt]) else STOP)
        self.steps.append((kind, [s for s, _ in entries]))
        return out

    def sample(self, logits, rows, samplers):
        return [logits[r] for r in rows]


def loop_for(backend, max_batch=8, context=64):
    return GenerationLoop(backend, max_batch=max_batch, context_length=context, default_stop_ids=(STOP,))


def req(prompt, max_tokens=16, stop=None):
    return GenerationRequest(list(prompt), max_tokens=max_tokens, sampler_config=SamplerConfig.greedy(),
                             stop_token_ids=stop)


def test_unequal_prompts_end_at_different_times():
    scripts = {(1, 2, 3): [10, 11, STOP], (4,): [20, 21, 22, 23, 24, STOP], (5, 6): [STOP]}
    be = ScriptedBackend(scripts)
    out = loop_for(be).run([req(p) for p in scripts])
    assert [r.token_ids for r in out] == [[10, 11], [20, 21, 22, 23, 24], []]
    assert [r.finish_reason for r in out] == ["stop", "stop", "stop"]
    assert [r.prompt_token_count for r in out] == [3, 1, 2]
    assert be.steps[0] == ("prefill", [0, 1, 2])
    assert be.steps[1] == ("decode", [0, 1]) and be.steps[3] == ("decode", [1])     # later steps are smaller
    assert not be.held and sorted(be.released) == [0, 1, 2]


def test_stop_token_is_neither_emitted_nor_fed():
    be = ScriptedBackend({(1,): [7, STOP, 8]})
    out = loop_for(be).run([req((1,))])
    assert out[0].token_ids == [7] and len(be.steps) == 2          # prefill + one decode; nothing after the stop


def test_budget_and_its_last_token_is_not_fed():
    be = ScriptedBackend({(1,): [7, 8, 9, 10]})
    out = loop_for(be).run([req((1,), max_tokens=3)])
    assert out[0].token_ids == [7, 8, 9] and out[0].finish_reason == "length"
    assert len(be.steps) == 3                                       # the third token needs no forward pass


def test_context_limit_and_long_prompts():
    be = ScriptedBackend({(1, 2, 3, 4): list(range(10, 40)), tuple(range(9)): [1]})
    out = loop_for(be, context=10).run([req((1, 2, 3, 4), max_tokens=30), req(tuple(range(9)))])
    # position = prompt + i must stay below context - 1 = 9: i = 0..5 emitted, the 6th ends it
    assert out[0].token_ids == list(range(10, 16)) and out[0].finish_reason == "context"
    assert out[1].finish_reason == "error" and "prompt too long (9 tokens, max 9)" in out[1].error
    assert out[1].token_ids == []


def test_batches_follow_one_another_and_slots_are_used_again():
    scripts = {(i,): [100 + i, STOP] for i in range(7)}
    be = ScriptedBackend(scripts, slots=3)
    out = loop_for(be, max_batch=3).run([req(p) for p in scripts])
    assert [r.token_ids for r in out] == [[100 + i] for i in range(7)]
    prefills = [s for s in be.steps if s[0] == "prefill"]
    assert [len(s[1]) for s in prefills] == [3, 3, 1]
    assert prefills[1][1] == [0, 1, 2] or sorted(prefills[1][1]) == [0, 1, 2]      # the same slots again
    assert not be.held


def test_batch_is_cut_where_the_cache_is_full():
    scripts = {(i, i): [50, STOP] for i in range(4)}
    be = ScriptedBackend(scripts, capacity=20)
    out = loop_for(be).run([req(p, max_tokens=6) for p in scripts])       # 8 tokens each: two fit
    assert [len(s[1]) for s in be.steps if s[0] == "prefill"] == [2, 2]
    assert all(r.token_ids == [50] for r in out)


def test_callback_can_stop_one_request():
    scripts = {(1,): [7, 8, 9, STOP], (2,): [3, 4, 5, STOP]}
    be = ScriptedBackend(scripts)
    seen = []

    def on_token(index, token):
        seen.append((index, token))
        return not (index == 0 and token == 8)

    out = loop_for(be).run([req(p) for p in scripts], on_token=on_token)
    assert out[0].token_ids == [7, 8] and out[0].finish_reason == "callback"
    assert out[1].token_ids == [3, 4, 5] and (1, 5) in seen


def test_request_stop_ids_override_and_zero_budget():
    be = ScriptedBackend({(1,): [7, 8, STOP], (2,): [1]})
    out = loop_for(be).run([req((1,), stop=[8]), req((2,), max_tokens=0)])
    assert out[0].token_ids == [7] and out[0].finish_reason == "stop"
    assert out[1].token_ids == [] and out[1].finish_reason == "length"


def test_slots_are_released_when_a_step_fails():
    class Failing(ScriptedBackend):
        def step(self, entries, want):
            if len(self.steps) == 1:
                raise RuntimeError("boom")
            return super().step(entries, want)

    be = Failing({(1,): [7, 8, 9]})
    with pytest.raises(RuntimeError):
        loop_for(be).run([req((1,))])
    assert not be.held
