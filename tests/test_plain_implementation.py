"""The plain implementation checked against itself and against properties the
reference's own diagnostics rely on (DiagnosticRunner.java:297-464)."""
import math

import pytest
import torch

import plain_llama as P
from helpers import TINY, make_model, random_tokens
from llmplayer_b200.parts.position import inverse_frequencies
from llmplayer_b200.parts.specs import Llama3Scaling, PositionSpec
from llmplayer_b200.sampling import JavaRandom


def test_rotation_at_position_zero_is_identity_and_shifts_cancel():
    inv = P.rope_inverse_frequencies(16, 10000.0)
    x = torch.randn(3, 2, 16, dtype=torch.float64)
    assert torch.equal(P.rope_rotate(x, torch.zeros(3, dtype=torch.long), inv), x)
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    def score(pq, pk):
        return float((P.rope_rotate(q, torch.tensor([pq]), inv) * P.rope_rotate(k, torch.tensor([pk]), inv)).sum())
    assert abs(score(5, 2) - score(25, 22)) < 1e-6          # only the distance matters


def test_pairings_agree_after_permuting_rows():
    inv = P.rope_inverse_frequencies(8, 500.0)
    x = torch.randn(4, 1, 8, dtype=torch.float64)
    pos = torch.arange(4)
    perm = torch.tensor([0, 4, 1, 5, 2, 6, 3, 7])           # split-half order -> neighbour order
    a = P.rope_rotate(x, pos, inv, "split_half")
    b = P.rope_rotate(x[..., perm], pos, inv, "interleaved")
    assert torch.allclose(a[..., perm], b, atol=1e-12)


def test_attention_at_position_zero_returns_the_value():
    q, k, v = torch.randn(1, 4, 8), torch.randn(1, 2, 8), torch.randn(1, 2, 8)
    out = P.attention(q, k, v, 0.3)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])


def test_window_drops_far_keys():
    T = 12
    q, k, v = torch.randn(T, 1, 4), torch.randn(T, 1, 4), torch.randn(T, 1, 4)
    full = P.attention(q, k, v, 0.5)
    win = P.attention(q, k, v, 0.5, window=5)
    assert torch.allclose(full[:5], win[:5]) and not torch.allclose(full[8], win[8])
    again = P.attention(q[8:9], k[4:9], v[4:9], 0.5)          # keys 4..8 only
    assert torch.allclose(win[8], again[0], atol=1e-6)


def test_causality_and_zero_layers(tmp_path):
    d = make_model(tmp_path, "B", dtype="float32")
    cfg, w = P.read_model(d)
    toks = random_tokens(9, 384, 3)
    full = P.forward(cfg, w, toks)
    assert torch.allclose(P.forward(cfg, w, toks[:5]), full[:5], atol=1e-12)
    zero = P.forward(cfg, w, toks[:1], layers=0)[0]
    e = w["model.embed_tokens.weight"].double()
    manual = w["lm_head.weight"].double() @ P.rms_norm(e[toks[0]], w["model.norm.weight"].double(), 1e-6)
    assert torch.allclose(zero, manual, atol=1e-12)


def test_float32_follows_float64(tmp_path):
    d = make_model(tmp_path, "A", dtype="float32")
    cfg, w = P.read_model(d)
    toks = random_tokens(20, 256, 1)
    a, b = P.forward(cfg, w, toks, dtype=torch.float64), P.forward(cfg, w, toks, dtype=torch.float32)
    assert float((a - b.double()).abs().max()) < 1e-5 * float(a.abs().max())


def test_llama3_frequencies_match_the_library_and_the_rule():
    scaling = {"factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    plain = P.rope_inverse_frequencies(32, 500000.0, scaling)
    spec = PositionSpec(head_dim=32, rotary_dim=32, theta=500000.0, scaling=Llama3Scaling(4.0, 1.0, 4.0, 64))
    assert torch.equal(plain, inverse_frequencies(spec))
    base = P.rope_inverse_frequencies(32, 500000.0)
    assert plain[0] == base[0]                                  # shortest wavelength (2 pi) is untouched
    assert abs(float(plain[-1]) * 4.0 / float(base[-1]) - 1) < 1e-6    # longest is stretched by the factor
    mid = [i for i in range(16) if 16.0 <= 2 * math.pi / float(base[i]) <= 64.0]
    assert mid and all(base[i] / 4 < plain[i] < base[i] for i in mid[1:-1])


def test_java_random_known_values():
    # the first nextFloat() of java.util.Random for seeds 42 and 0
    assert abs(JavaRandom(42).next_float() - 0.7275637) < 1e-7
    assert abs(JavaRandom(0).next_float() - 0.73096776) < 1e-7
    assert P.JavaRandom(42).next_float() == JavaRandom(42).next_float()


def test_plain_sampler_stages():
    logits = torch.tensor([1.0, 3.0, 3.0, 2.0, -1.0])
    assert P.PlainSampler(temperature=0.0, repetition_penalty=1.0).sample(logits) == 1     # first maximum
    s = P.PlainSampler(temperature=0.0, repetition_penalty=2.0)
    assert s.sample(logits) == 1 and s.sample(logits) == 2          # token 1 now counts 1.5
    s = P.PlainSampler(temperature=1.0, top_k=2, top_p=1.0, repetition_penalty=1.0, seed=7)
    assert {s.sample(logits) for _ in range(50)} == {1, 2}          # ties at the threshold both survive
    s = P.PlainSampler(temperature=1.0, top_k=0, top_p=0.5, repetition_penalty=1.0, seed=7)
    assert {s.sample(logits) for _ in range(50)} <= {1, 2}
    s = P.PlainSampler(temperature=1.0, top_k=0, top_p=1.0, min_p=0.9, repetition_penalty=1.0, seed=3)
    assert {s.sample(logits) for _ in range(50)} == {1, 2}
