"""Generation through the Python entry point: greedy against the plain implementation,
stop tokens, batches that follow one another, seeded temperature sampling."""
import pytest
import torch

import plain_llama as P
from helpers import TINY, make_model, random_tokens, tolerance

pytestmark = pytest.mark.gpu


def prompts_for(name, lengths, seed=0):
    vocab = TINY[name][0]["vocab_size"]
    return [random_tokens(n, vocab, seed=seed + i) for i, n in enumerate(lengths)]


def check_greedy_chain(model_dir, prompt, generated, dtype, config=None):
    """Every generated token must be the plain implementation's argmax at its place, up to the
    dtype's tolerance on the logits (in float32 that means: the same token)."""
    cfg, w = P.read_model(model_dir)
    seq = list(prompt) + list(generated)
    logits = P.forward(cfg, w, seq, dtype=torch.float64)
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        slack = 2 * tolerance(dtype, config) * float(row.abs().max())
        assert float(row[tok]) >= float(row.max()) - slack, (i, tok, int(row.argmax()))
        if dtype == "float32":
            assert tok == P.argmax_first(row)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,steps", [("A", [5, 9, 13], 8), ("B", [1, 7, 16, 30], 12)])
def test_greedy_generation_through_the_entry_point(tmp_path, name, lengths, steps, dtype):
    from llmplayer_b200 import Engine, SamplerConfig
    model_dir = make_model(tmp_path, name, dtype=dtype)
    prompts = prompts_for(name, lengths)
    eng = Engine.load(model_dir, dtype=dtype, context_length=128, max_batch=len(prompts))
    out = eng.generate(prompts, SamplerConfig.greedy(), max_tokens=steps, stop_token_ids=())
    assert [r.finish_reason for r in out] == ["length"] * len(prompts)
    for p, r in zip(prompts, out):
        assert r.token_count == steps and r.prompt_token_count == len(p)
        check_greedy_chain(model_dir, p, r.token_ids, dtype, name)
    assert eng.cache.slots.num_held == 0 and eng.cache.free_pages() == [eng.cache.num_pages]
    stats = eng.last_generation_stats
    assert stats.generated_tokens == steps * len(prompts) and stats.decode_tokens_per_second > 0


def test_stop_token_ends_one_sequence_while_others_go_on(tmp_path):
    from llmplayer_b200 import Engine, SamplerConfig
    model_dir = make_model(tmp_path, "A", dtype="float32")
    prompts = prompts_for("A", [6, 11, 4], seed=20)
    eng = Engine.load(model_dir, dtype="float32", context_length=128, max_batch=3)
    free = eng.generate(prompts, SamplerConfig.greedy(), max_tokens=10, stop_token_ids=())
    stop = free[1].token_ids[3]
    cut = eng.generate(prompts, SamplerConfig.greedy(), max_tokens=10, stop_token_ids=[stop])
    for a, b in zip(free, cut):
        want = a.token_ids[:a.token_ids.index(stop)] if stop in a.token_ids else a.token_ids
        assert b.token_ids == want
        assert b.finish_reason == ("stop" if stop in a.token_ids else "length")
    assert cut[1].token_count <= 3


def test_more_requests_than_slots_run_as_batches_one_after_another(tmp_path):
    from llmplayer_b200 import Engine, SamplerConfig
    model_dir = make_model(tmp_path, "B", dtype="float32")
    prompts = prompts_for("B", [3, 40, 9, 1, 22, 17, 5], seed=40)
    eng = Engine.load(model_dir, dtype="float32", context_length=64, max_batch=3)
    batched = eng.generate(prompts, SamplerConfig.greedy(), max_tokens=6, stop_token_ids=())
    assert eng.last_generation_stats.batches == 3
    single = Engine.load(model_dir, dtype="float32", context_length=64, max_batch=1)
    for p, r in zip(prompts, batched):
        alone = single.generate([p], SamplerConfig.greedy(), max_tokens=6, stop_token_ids=())[0]
        assert alone.token_ids == r.token_ids
        check_greedy_chain(model_dir, p, r.token_ids, "float32")


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(tmp_path):
    from llmplayer_b200 import Engine, SamplerConfig
    from llmplayer_b200.engine.generate import GenerationRequest
    model_dir = make_model(tmp_path, "B", dtype="float32")
    prompts = prompts_for("B", [1, 7, 16, 30], seed=60)
    eng = Engine.load(model_dir, dtype="float32", context_length=128, max_batch=4)
    cfg = SamplerConfig(temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=1)
    a = eng.generate(prompts, cfg, max_tokens=12, stop_token_ids=())
    b = eng.generate(prompts, cfg, max_tokens=12, stop_token_ids=())
    assert [r.token_ids for r in a] == [r.token_ids for r in b]
    alone = eng.generate([prompts[2]], cfg, max_tokens=12, stop_token_ids=())[0]
    assert alone.token_ids == a[2].token_ids
    other = eng.generate(prompts, cfg.with_seed(2), max_tokens=12, stop_token_ids=())
    assert [r.token_ids for r in other] != [r.token_ids for r in a]
    # the plain sampler, fed the plain logits along the engine's own sequence, draws the same tokens
    cfg_plain, w = P.read_model(model_dir)
    ps = P.PlainSampler(temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=1)
    seq = list(prompts[1])
    for tok in a[1].token_ids:
        assert ps.sample(P.forward(cfg_plain, w, seq, dtype=torch.float64)[-1]) == tok
        seq.append(tok)


def test_prompt_too_long_is_an_error_response(tmp_path):
    from llmplayer_b200 import Engine, SamplerConfig
    model_dir = make_model(tmp_path, "A", dtype="float32")
    eng = Engine.load(model_dir, dtype="float32", context_length=16, max_batch=2)
    out = eng.generate([list(range(15)), [1, 2, 3]], SamplerConfig.greedy(), max_tokens=40, stop_token_ids=())
    assert out[0].finish_reason == "error" and "prompt too long" in out[0].error
    assert out[1].finish_reason == "context" and out[1].token_count == 16 - 1 - 3 + 1


def test_native_host_loop_equals_stepping_from_python(tmp_path):
    """Greedy decoding through the native host loop (a captured graph per step with upload, argmax and
    read-back inside, several quiet steps per call) must give what the loop gives when every step goes
    through ``Engine.step`` and ``Engine.sample``: across page boundaries, with a stop token that ends one
    sequence in the middle of a run, with unequal budgets, and with a callback (one step per call)."""
    from llmplayer_b200 import Engine, SamplerConfig
    from llmplayer_b200.engine.generate import GenerationRequest
    model_dir = make_model(tmp_path, "C", dtype="bfloat16")
    prompts = prompts_for("C", [50, 3, 61], seed=80)
    fast = Engine.load(model_dir, dtype="bfloat16", context_length=512, max_batch=3)
    slow = Engine.load(model_dir, dtype="bfloat16", context_length=512, max_batch=3, host_loop=False, graphs=False)
    steps = 90
    ref = slow.generate(prompts, SamplerConfig.greedy(), max_tokens=steps + 1, stop_token_ids=())
    got = fast.generate(prompts, SamplerConfig.greedy(), max_tokens=steps + 1, stop_token_ids=())
    assert fast.last_generation_stats.decode_steps == steps
    assert any(e.get("graph") is not None for e in fast._fused.values()), "the captured step never ran"
    for p, r, g in zip(prompts, ref, got):
        assert g.finish_reason == "length" and g.token_count == steps + 1
        check_greedy_chain(model_dir, p, g.token_ids, "bfloat16", "C")
        check_greedy_chain(model_dir, p, r.token_ids, "bfloat16", "C")
    # a stop token in the middle: the 30th token of the second sequence; budgets differ per request
    stop = got[1].token_ids[29]
    first_hit = [r.token_ids.index(stop) if stop in r.token_ids else None for r in got]
    requests = [GenerationRequest(p, max_tokens=m, sampler_config=SamplerConfig.greedy(), stop_token_ids=(stop,))
                for p, m in zip(prompts, (70, 91, 20))]
    again = fast.generate(requests)
    for r, full, hit, budget in zip(again, got, first_hit, (70, 91, 20)):
        if hit is not None and hit < budget:
            assert r.finish_reason == "stop" and r.token_ids == full.token_ids[:hit]
        else:
            assert r.finish_reason == "length" and r.token_ids == full.token_ids[:budget]
    # with a callback every token passes through the interpreter before the next step
    seen = []
    called = fast.generate(prompts, SamplerConfig.greedy(), max_tokens=40, stop_token_ids=(),
                           on_token=lambda i, t: seen.append((i, t)))
    assert [r.token_ids for r in called] == [g.token_ids[:40] for g in got]
    assert len(seen) == 3 * 40
    assert fast.cache.slots.num_held == 0 and slow.cache.slots.num_held == 0


def test_native_loop_with_samplers_equals_stepping_from_python(tmp_path):
    """Temperature / top-k / top-p sampling with a repetition penalty through the native host loop (the sampler's
    generator and its window of recent tokens kept by csrc/host_loop.cu, the sampler block fetched inside the
    captured step) must give, token for token, what ``Engine.step`` + ``Engine.sample`` give from the interpreter:
    same seeds, unequal prompts and budgets, a greedy row with a penalty among them, a stop token on the way, and
    and one sequence whose window of recent tokens is 64 long, so that its oldest tokens leave the window on the
    way (seeds differ per request, so a generator that was advanced wrongly shows)."""
    from llmplayer_b200 import Engine, SamplerConfig
    from llmplayer_b200.engine.generate import GenerationRequest
    model_dir = make_model(tmp_path, "C", dtype="bfloat16")
    prompts = prompts_for("C", [50, 3, 61, 20], seed=81)
    configs = [SamplerConfig(temperature=0.8, top_k=20, top_p=0.9, repetition_penalty=1.3, seed=11),
               SamplerConfig(temperature=1.1, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=12),
               SamplerConfig(temperature=0.0, top_k=1, top_p=1.0, repetition_penalty=1.2, seed=13),
               SamplerConfig(temperature=0.7, top_k=40, top_p=0.9, repetition_penalty=1.5, seed=14, min_p=0.02,
                             dry_range=64)]
    fast = Engine.load(model_dir, dtype="bfloat16", context_length=512, max_batch=4)
    slow = Engine.load(model_dir, dtype="bfloat16", context_length=512, max_batch=4, host_loop=False)

    def requests(budgets, stop=()):
        return [GenerationRequest(p, max_tokens=m, sampler_config=c, stop_token_ids=stop)
                for p, m, c in zip(prompts, budgets, configs)]

    ref = slow.generate(requests((90, 91, 70, 150)))
    got = fast.generate(requests((90, 91, 70, 150)))
    assert any(e.get("graph") is not None for e in fast._fused.values()), "the captured step never ran"
    assert any(len(k) > 4 and k[4] == "sampled" for k in fast._fused), "the sampled form of the captured step never ran"
    for r, g in zip(ref, got):
        assert g.finish_reason == r.finish_reason == "length"
        assert g.token_ids == r.token_ids
    assert len({tuple(g.token_ids[:20]) for g in got}) == 4          # the rows really differ
    # a stop token that the first sequence meets on the way
    stop = (got[0].token_ids[33],)
    ref = slow.generate(requests((90, 91, 70, 40), stop))
    got = fast.generate(requests((90, 91, 70, 40), stop))
    assert [g.finish_reason for g in got] == [r.finish_reason for r in ref]
    assert got[0].finish_reason == "stop"
    assert [g.token_ids for g in got] == [r.token_ids for r in ref]
    assert fast.cache.slots.num_held == 0 and slow.cache.slots.num_held == 0
