"""The device sampler against the plain restatement of the reference's sampler."""
import pytest
import torch

import plain_llama as P
from llmplayer_b200.sampling import BatchSampler, SamplerConfig, SequenceSampler

pytestmark = pytest.mark.gpu

CONFIGS = [
    dict(temperature=0.0, top_k=1, top_p=1.0, repetition_penalty=1.0),
    dict(temperature=0.0, top_k=40, top_p=0.9, repetition_penalty=1.3),
    dict(temperature=0.8, top_k=0, top_p=1.0, repetition_penalty=1.0),
    dict(temperature=0.7, top_k=40, top_p=0.9, repetition_penalty=1.1),          # the reference's defaults
    dict(temperature=1.3, top_k=0, top_p=0.8, repetition_penalty=1.0),
    dict(temperature=1.0, top_k=5000, top_p=0.95, repetition_penalty=1.2),       # more survivors than fit on chip
    dict(temperature=1.0, top_k=0, top_p=1.0, min_p=0.05, repetition_penalty=1.0),
    dict(temperature=0.9, top_k=50, top_p=1.0, mirostat=2, mirostat_tau=3.0, mirostat_eta=0.2, repetition_penalty=1.0),
    dict(temperature=1.0, top_k=0, top_p=1.0, mirostat=2, repetition_penalty=1.0),
    dict(temperature=0.8, top_k=20, top_p=0.9, repetition_penalty=1.1, dry_multiplier=0.8, dry_allowed_length=1,
         dry_range=16),
    dict(temperature=1.1, top_k=900, top_p=0.97, repetition_penalty=1.0),        # many candidates on chip
    dict(temperature=1.2, top_k=700, top_p=1.0, mirostat=2, mirostat_tau=6.0, repetition_penalty=1.0),
]


def make_logits(V, steps, seed, spread):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(steps, V, generator=g) * spread
    x[:, 7] = x[:, 11]                       # exact ties
    x[::3, 5] = x[::3].max(dim=1).values     # ... also at the maximum
    return x


@pytest.mark.parametrize("V,spread", [(1000, 3.0), (5003, 1.5), (128256, 2.0)])
def test_batched_sampler_follows_the_plain_one(V, spread):
    steps = 24 if V < 100000 else 6
    dev = torch.device("cuda:0")
    configs = CONFIGS if V < 100000 else CONFIGS[:8]
    logits = [make_logits(V, steps, seed=i, spread=spread) for i in range(len(configs))]
    if V < 100000:
        for x in logits:                     # a small alphabet in the lead, so that tokens repeat
            x[:, :6] += 3.0 * spread
    plain = [P.PlainSampler(seed=100 + i, **c) for i, c in enumerate(configs)]
    ours = [SequenceSampler(SamplerConfig(seed=100 + i, **c)) for i, c in enumerate(configs)]
    batch = BatchSampler(V, dev)
    mismatches = []
    for t in range(steps):
        rows = torch.stack([x[t] for x in logits]).to(dev)
        got = batch.sample(rows, list(range(len(configs))), ours)
        want = [p.sample(x[t]) for p, x in zip(plain, logits)]
        for i, (a, b) in enumerate(zip(got, want)):
            if a != b:
                mismatches.append((t, i, a, b))
                # keep both histories alike so that later steps stay comparable
                ours[i].recent[-1] = b
    assert not mismatches, mismatches


@pytest.mark.parametrize("V", [5003, 40000])
def test_top_k_among_many_equal_values(V):
    """Rows whose values repeat: the k-th largest has many equals, in one slice of the row or in all of them,
    up to a row of one value only, where top-k keeps the whole vocabulary."""
    dev = torch.device("cuda:0")
    steps = 6
    g = torch.Generator().manual_seed(77)
    base = torch.randn(steps, V, generator=g) * 2.0
    rows = [torch.round(base), torch.round(base * 4) / 4, torch.full((steps, V), 0.5),
            torch.where(torch.arange(V) < V // 7, torch.round(base) + 2.0, base)]
    configs = [dict(temperature=0.9, top_k=40, top_p=0.9, repetition_penalty=1.1),
               dict(temperature=1.0, top_k=64, top_p=1.0, repetition_penalty=1.0),
               dict(temperature=0.8, top_k=30, top_p=0.95, repetition_penalty=1.2),
               dict(temperature=1.1, top_k=50, top_p=0.9, mirostat=2, repetition_penalty=1.0)]
    plain = [P.PlainSampler(seed=7 + i, **c) for i, c in enumerate(configs)]
    ours = [SequenceSampler(SamplerConfig(seed=7 + i, **c)) for i, c in enumerate(configs)]
    batch = BatchSampler(V, dev)
    mismatches = []
    for t in range(steps):
        got = batch.sample(torch.stack([x[t] for x in rows]).to(dev), list(range(len(rows))), ours)
        want = [p.sample(x[t]) for p, x in zip(plain, rows)]
        for i, (a, b) in enumerate(zip(got, want)):
            if a != b:
                mismatches.append((t, i, a, b))
                ours[i].recent[-1] = b
    assert not mismatches, mismatches


@pytest.mark.parametrize("V,spread", [(5003, 6.0), (128256, 5.0), (128256, 9.0)])
def test_top_p_without_top_k_on_peaked_rows(V, spread):
    """Rows as a trained model gives them, with most of the mass on a few tokens: the cut of top-p lies among
    the largest values, which are then carried on alone. The widest spread leaves probabilities of zero."""
    dev = torch.device("cuda:0")
    steps = 8
    configs = [dict(temperature=1.0, top_k=0, top_p=0.9, repetition_penalty=1.0),
               dict(temperature=0.7, top_k=0, top_p=0.95, repetition_penalty=1.1),
               dict(temperature=1.2, top_k=0, top_p=0.6, min_p=0.001, repetition_penalty=1.0),
               dict(temperature=1.0, top_k=0, top_p=0.9, mirostat=2, mirostat_tau=4.0, repetition_penalty=1.0),
               dict(temperature=1.0, top_k=5000, top_p=0.9, repetition_penalty=1.0)]
    logits = [make_logits(V, steps, seed=40 + i, spread=spread) for i in range(len(configs))]
    plain = [P.PlainSampler(seed=3 + i, **c) for i, c in enumerate(configs)]
    ours = [SequenceSampler(SamplerConfig(seed=3 + i, **c)) for i, c in enumerate(configs)]
    batch = BatchSampler(V, dev)
    mismatches = []
    for t in range(steps):
        got = batch.sample(torch.stack([x[t] for x in logits]).to(dev), list(range(len(configs))), ours)
        want = [p.sample(x[t]) for p, x in zip(plain, logits)]
        for i, (a, b) in enumerate(zip(got, want)):
            if a != b:
                mismatches.append((t, i, a, b))
                ours[i].recent[-1] = b
    assert not mismatches, mismatches


def test_draws_do_not_depend_on_the_batch():
    dev = torch.device("cuda:0")
    V = 777
    x = make_logits(V, 10, seed=5, spread=2.0)
    cfg = SamplerConfig(temperature=0.9, top_k=30, top_p=0.9, repetition_penalty=1.1, seed=42)
    alone = SequenceSampler(cfg)
    batch = BatchSampler(V, dev)
    a = [batch.sample(x[t:t + 1].to(dev), [0], [alone])[0] for t in range(10)]
    together = SequenceSampler(cfg)
    other = SequenceSampler(SamplerConfig(temperature=1.5, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=1))
    y = make_logits(V, 10, seed=6, spread=2.0)
    b = []
    for t in range(10):
        rows = torch.stack([y[t], x[t]]).to(dev)
        b.append(batch.sample(rows, [0, 1], [other, together])[1])
    assert a == b


@pytest.mark.parametrize("B,V", [(1, 1000), (8, 128256), (64, 5003)])
def test_batched_argmax_takes_the_first_maximum(B, V):
    from llmplayer_b200.kernels import ops
    x = make_logits(V, B, seed=B, spread=2.0).to("cuda:0")
    x[:, V - 1] = x.max(dim=1).values          # a tie with the maximum at the far end must lose
    out = torch.empty(B, dtype=torch.int32, device="cuda:0")
    ops.argmax(x, torch.empty(64 * B, device="cuda:0"), out)
    assert out.tolist() == [P.argmax_first(row) for row in x.cpu()]
