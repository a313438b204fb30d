"""The sampler's state on the host (recent tokens, logit edits, draws, mirostat's mu) against the plain sampler.

What depends on the logits runs on the device and is compared there token by token; here the
edits that the host prepares are applied to a row with the kernel's formula and compared with
the row as the plain sampler edits it.
"""
import math

import torch

import plain_llama as P
from llmplayer_b200.sampling import SamplerConfig, SequenceSampler


def apply_edits(logits, edits):
    """The kernel's edit of a row: subtract, then divide a positive value by the factor, multiply another."""
    out = logits.clone()
    for tok, sub, fac in edits:
        v = out[tok] - torch.tensor(sub, dtype=torch.float32)
        f = torch.tensor(fac, dtype=torch.float32)
        out[tok] = v / f if v > 0 else v * f
    return out


def plain_edited(sampler, logits):
    """The row as the plain sampler has it after its DRY and repetition penalties."""
    p = logits.clone()
    c = sampler.c
    if c["dry_multiplier"] > 0:
        sampler._dry(p)
    if c["repetition_penalty"] != 1.0:
        r = torch.tensor(c["repetition_penalty"], dtype=torch.float32)
        for tok in sampler.recent:
            p[tok] = p[tok] / r if p[tok] > 0 else p[tok] * r
    return p


def test_repetition_penalty_counts_every_occurrence():
    s = SequenceSampler(SamplerConfig(temperature=0.8, repetition_penalty=1.3, seed=1))
    for tok in (5, 9, 5, 5, 2):
        s.accept(tok, 0.5)
    edits = {tok: (sub, fac) for tok, sub, fac in s.logit_edits()}
    assert set(edits) == {2, 5, 9}
    assert edits[5][0] == 0.0 and abs(edits[5][1] - 1.3 ** 3) < 1e-12
    assert abs(edits[9][1] - 1.3) < 1e-12 and abs(edits[2][1] - 1.3) < 1e-12
    assert [tok for tok, _, _ in s.logit_edits()] == [2, 5, 9]          # in token order, each once


def test_no_edits_without_penalties_and_none_before_the_first_token():
    assert SequenceSampler(SamplerConfig(temperature=0.8, repetition_penalty=1.3)).logit_edits() == []
    s = SequenceSampler(SamplerConfig(temperature=0.8, repetition_penalty=1.0))
    for tok in (1, 2, 3):
        s.accept(tok, 1.0)
    assert s.logit_edits() == []


def test_edits_follow_the_plain_sampler_over_a_history():
    g = torch.Generator().manual_seed(3)
    V = 50
    config = dict(temperature=0.9, top_k=0, top_p=1.0, repetition_penalty=1.15, dry_multiplier=0.8, dry_base=1.75,
                  dry_allowed_length=2, dry_range=24)
    ours = SequenceSampler(SamplerConfig(seed=5, **config))
    plain = P.PlainSampler(seed=5, **config)
    # a history with repeated runs, so that the DRY penalty finds suffixes of several lengths
    history = [3, 4, 5, 6, 3, 4, 5, 7, 8, 3, 4, 5, 6, 3, 4, 9, 3, 4, 5] + torch.randint(0, 10, (60,), generator=g).tolist()
    for t, tok in enumerate(history):
        logits = torch.randn(V, generator=g) * 3
        got = apply_edits(logits, ours.logit_edits())
        want = plain_edited(plain, logits)
        assert torch.allclose(got, want, rtol=2e-6, atol=1e-6), (t, (got - want).abs().max())
        ours.accept(tok, 0.5)
        plain._remember(tok)
    assert ours.recent == plain.recent and len(ours.recent) == max(64, 24)


def test_draws_are_javas_and_greedy_takes_none():
    s = SequenceSampler(SamplerConfig(temperature=0.7, seed=42))
    ref = P.JavaRandom(42)
    assert [s.draw() for _ in range(5)] == [ref.next_float() for _ in range(5)]
    greedy = SequenceSampler(SamplerConfig.greedy())
    assert greedy.draw() == 0.0 and greedy.mirostat_threshold() == -1.0


def test_mirostat_threshold_follows_the_observed_surprise():
    c = dict(temperature=1.0, mirostat=2, mirostat_tau=4.0, mirostat_eta=0.25)
    s = SequenceSampler(SamplerConfig(**c))
    assert s.mirostat_threshold() == math.pow(2.0, -8.0)             # mu starts at 2 tau
    mu = 8.0
    for prob in (0.5, 0.01, 0.9, 1.0):
        s.accept(1, prob)
        mu -= 0.25 * (-math.log2(prob) - 4.0)
        assert abs(s.mirostat_threshold() - math.pow(2.0, -mu)) < 1e-12
    off = SequenceSampler(SamplerConfig(temperature=1.0, mirostat=0))
    assert off.mirostat_threshold() == -1.0
