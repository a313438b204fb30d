"""Generality of the parts, shown with toys defined here and registered from outside the
package: a mixer with state of its own, layers that differ (a window here, all keys there),
a layer that runs twice, and a run that attends over another run's cache. The toy model is
stepped whole, in chunks and in batches with slot re-use, and compared with a plain
restatement written in this file."""
import json
import math
import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import pytest
import torch

import plain_llama as P
from helpers import assert_close, random_tokens

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- a toy mixer
@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    decay: float
    gain: str
    kind: str = "toy_decay"


def make_decay_mixer():
    from llmplayer_b200.cache import StateRequest
    from llmplayer_b200.parts.base import Part
    from llmplayer_b200.parts.specs import GAIN, TensorSpec

    class DecayMixer(Part):
        """state <- decay * state + x_t;  residual_t += state * gain. One float32 row per sequence."""

        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            return {self.spec.gain: TensorSpec((self.spec.hidden_size,), GAIN)}

        def load(self, tensors, runtime):
            super().load(tensors, runtime)
            self.gain = runtime.gain(tensors[self.spec.gain])

        def cache_request(self):
            return StateRequest((self.spec.hidden_size,), torch.float32)

        def forward(self, ctx, cache, x, residual):
            for seq in ctx.sequences:                       # tokens of a sequence in order
                state = cache.rows[seq.slot]
                for t in range(seq.start, seq.start + seq.num_new):
                    state.mul_(self.spec.decay).add_(x[t].float())
                    residual[t] += state * self.gain

    return DecayMixer


# ----------------------------------------------------------------------------- a toy architecture
def make_toy_config():
    from llmplayer_b200.config.registry import ArchitectureConfig
    from llmplayer_b200.parts.specs import (
        AttentionSpec, BlockSpec, EmbeddingSpec, HeadSpec, ModelLayout, NormSpec, PositionSpec, ScheduleEntry, SwiGLUSpec,
    )

    @dataclass(frozen=True)
    class ToyConfig(ArchitectureConfig):
        hidden_size: int
        vocab_size: int
        window: int
        architecture = "ToyForTest"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["hidden_size"], raw["vocab_size"], raw["window"])

        def to_dict(self):
            return {"architectures": ["ToyForTest"], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                    "window": self.window}

        def max_positions(self):
            return 512

        def layout(self):
            d = self.hidden_size

            def attention(i, heads, kv, hd, window=None, shares=False, theta=10000.0, rotary=None):
                p = f"layers.{i}."
                return AttentionSpec(
                    hidden_size=d, num_heads=heads, num_kv_heads=kv, head_dim=hd, scale=1.0 / math.sqrt(hd),
                    position=PositionSpec("rope", hd, rotary or hd, theta), q=p + "q", o=p + "o",
                    k=None if shares else p + "k", v=None if shares else p + "v", window=window, shares_kv=shares)

            def block(i, mixer, F):
                p = f"layers.{i}."
                return BlockSpec(NormSpec(d, 1e-5, p + "n1"), mixer, NormSpec(d, 1e-6, p + "n2"),
                                 SwiGLUSpec(d, F, p + "g", p + "u", p + "d"))

            layers = (
                block(0, attention(0, 4, 2, 16, window=self.window), 96),               # a window of keys
                block(1, DecaySpec(d, 0.9, "layers.1.gain"), 64),                       # state of its own
                block(2, attention(2, 2, 1, 32, theta=500.0, rotary=16), 80),           # all keys, other geometry
                block(3, attention(3, 4, 1, 32, shares=True, theta=500.0, rotary=16), 64),   # no keys of its own
            )
            schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(0),
                        ScheduleEntry(3, reads_cache_of=2), ScheduleEntry(1))
            return ModelLayout(EmbeddingSpec(self.vocab_size, d, "embed"), layers,
                               HeadSpec(self.vocab_size, d, NormSpec(d, 1e-5, "norm"), "head"), schedule)

    return ToyConfig


@pytest.fixture()
def toy():
    from llmplayer_b200.config import register_architecture, unregister_architecture
    from llmplayer_b200.parts import MIXERS
    MIXERS.register("toy_decay", make_decay_mixer(), replace=True)
    cfg = make_toy_config()
    register_architecture("ToyForTest", cfg, replace=True)
    yield cfg
    unregister_architecture("ToyForTest")
    MIXERS.unregister("toy_decay")


# ----------------------------------------------------------------------------- its plain restatement
def plain_toy(w, tokens, window):
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)]
    kept = {}

    def attn(i, x, heads, kv, hd, theta, rotary, win, run, shared_from=None):
        p = f"layers.{i}."
        inv = P.rope_inverse_frequencies(rotary, theta)
        q = P.rope_rotate((x @ w[p + "q"].T).reshape(T, heads, hd), pos, inv)
        if shared_from is None:
            k = P.rope_rotate((x @ w[p + "k"].T).reshape(T, kv, hd), pos, inv)
            v = (x @ w[p + "v"].T).reshape(T, kv, hd)
            kept[run] = (k, v)
        else:
            k, v = kept[shared_from]
        o = P.attention(q, k, v, 1.0 / math.sqrt(hd), window=win, q_positions=pos)
        return o.reshape(T, heads * hd) @ w[p + "o"].T

    def decay(x, state):
        out = torch.zeros_like(x)
        for t in range(T):
            state = 0.9 * state + x[t]
            out[t] = state * w["layers.1.gain"]
        return out

    def ffn(i, x):
        p = f"layers.{i}."
        return P.swiglu(P.rms_norm(x, w[p + "n2"], 1e-6), w[p + "g"], w[p + "u"], w[p + "d"])

    def norm1(i, x):
        return P.rms_norm(x, w[f"layers.{i}.n1"], 1e-5)

    d = x.shape[1]
    for run, layer in enumerate([0, 1, 2, 0, 3, 1]):
        h = norm1(layer, x)
        if layer == 0:
            x = x + attn(0, h, 4, 2, 16, 10000.0, 16, window, run)
        elif layer == 1:
            x = x + decay(h, torch.zeros(d, dtype=torch.float64))      # each run has a state of its own
        elif layer == 2:
            x = x + attn(2, h, 2, 1, 32, 500.0, 16, None, run)
        else:
            x = x + attn(3, h, 4, 1, 32, 500.0, 16, None, run, shared_from=2)
        x = x + ffn(layer, x)
    return P.rms_norm(x, w["norm"], 1e-5) @ w["head"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_is_registered_built_and_stepped(tmp_path, toy, dtype):
    from llmplayer_b200 import Engine
    from llmplayer_b200.cache import KVRequest, StateRequest
    from llmplayer_b200.weights import write_random_model
    window = 20
    model_dir = str(tmp_path / "toy")
    write_random_model(toy(hidden_size=64, vocab_size=97, window=window), 3, model_dir, dtype=dtype, std=0.08)
    assert json.load(open(os.path.join(model_dir, "config.json")))["architectures"] == ["ToyForTest"]
    weights = P.read_safetensors(os.path.join(model_dir, "model.safetensors"))
    assert "layers.3.k" not in weights and "layers.1.gain" in weights

    eng = Engine.load(model_dir, dtype=dtype, max_tokens=6 * 128, max_slots=4)
    requests = eng.model.cache_requests()
    assert [type(r) for r in requests] == [KVRequest, StateRequest, KVRequest, KVRequest, type(None), StateRequest]
    assert len(eng.cache.groups) == 2                           # windowed runs and full runs: storage of their own
    assert {g.request.window for g in eng.cache.groups} == {window, None}
    assert eng.cache.view(4) is None and eng.model.cache_owner(4) == 2

    seqs = [random_tokens(n, 97, seed=n) for n in (5, 90, 33, 1, 70)]
    refs = [plain_toy(weights, s, window) for s in seqs]

    # whole
    for s, ref in zip(seqs, refs):
        slot = eng.acquire()
        got = eng.step([(slot, s)], [list(range(len(s)))]).cpu()
        eng.release(slot)
        assert_close(got, ref, dtype, "toy whole", config="toy")

    # a prefix, then a chunk, then one by one
    s, ref = seqs[1], refs[1]
    slot = eng.acquire()
    rows = [eng.step([(slot, s[:40])], [list(range(40))]).cpu().clone(),
            eng.step([(slot, s[40:70])], [list(range(30))]).cpu().clone()]
    rows += [eng.step([(slot, [t])], [[0]]).cpu().clone() for t in s[70:]]
    eng.release(slot)
    assert_close(torch.cat(rows), ref, dtype, "toy in steps", config="toy")

    # batches of unequal lengths, shorter ones end earlier, slots are used again
    for group in ([0, 1, 2], [3, 4, 0]):
        slots = {i: eng.acquire() for i in group}
        got = {i: [] for i in group}
        fed = {i: max(1, len(seqs[i]) // 2) for i in group}
        out = eng.step([(slots[i], seqs[i][:fed[i]]) for i in group], [list(range(fed[i])) for i in group]).cpu()
        at = 0
        for i in group:
            got[i].append(out[at:at + fed[i]].clone())
            at += fed[i]
        live = [i for i in group if fed[i] < len(seqs[i])]
        for i in group:
            if i not in live:
                eng.release(slots[i])
        while live:
            out = eng.step([(slots[i], [seqs[i][fed[i]]]) for i in live], [[0] for _ in live]).cpu()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1].clone())
                fed[i] += 1
            for i in [i for i in live if fed[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if fed[i] < len(seqs[i])]
        for i in group:
            assert_close(torch.cat(got[i]), refs[i], dtype, f"toy batch, request {i}", config="toy")
    assert eng.cache.slots.num_held == 0
    assert all(g.pages.pool.num_free == g.pages.pool.count for g in eng.cache.groups)


def test_unknown_kinds_are_refused():
    from llmplayer_b200.errors import ConfigError
    from llmplayer_b200.parts import MIXERS
    with pytest.raises(ConfigError, match="unknown mixer kind 'nope'.*attention"):
        MIXERS.build(DecaySpec(8, 0.5, "g", kind="nope"))


# ----------------------------------------------------------------------------- more toys: a position encoding
# that is no rotation, a feed-forward with a router, and a mixer whose state is indexed on the device
@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    router: str
    gate: str
    up: str
    down: str
    kind: str = "toy_routed"


@dataclass(frozen=True)
class DeviceDecaySpec:
    hidden_size: int
    decay: float
    gain: str
    kind: str = "toy_decay_device"


def make_more_toys():
    from llmplayer_b200.cache import StateRequest
    from llmplayer_b200.parts.base import Part
    from llmplayer_b200.parts.specs import GAIN, MATRIX, TensorSpec

    class DistanceDecay(Part):
        """Queries are multiplied by base^(position / span), keys divided by it, feature by feature: a score then
        carries base^((p_query - p_key) / span). Not a rotation, so the kernels cannot apply it on the way:
        ``rotation()`` is None and ``apply`` changes the projection in place."""
        capture_safe = True          # reads positions from the device only

        def __init__(self, spec):
            self.spec = spec         # a PositionSpec: theta is the base, rotary_dim the span

        def rotation(self):
            return None

        def apply(self, ctx, qkv, *, num_heads, num_kv_heads, head_dim):
            # base^(position / span) from device tensors and host scalars only (nothing is copied: capturable)
            factor = torch.exp2(ctx.positions.to(torch.float32) * (math.log2(self.spec.theta) / self.spec.rotary_dim))[:, None]
            nq = num_heads * head_dim
            qkv[:, :nq] *= factor
            if num_kv_heads:
                qkv[:, nq:nq + num_kv_heads * head_dim] /= factor

    class RoutedFeedForward(Part):
        """Each token goes to the one expert with the largest router logit (float32) and gets that expert's gated
        feed-forward, weighted by the softmax probability of the choice. Plain torch on the device: a toy, which
        runs every expert over every token and keeps the chosen one's result (no shape depends on the routing,
        so a step can be captured)."""
        capture_safe = True

        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            s = self.spec
            return {s.router: TensorSpec((s.num_experts, s.hidden_size), MATRIX),
                    s.gate: TensorSpec((s.num_experts * s.intermediate_size, s.hidden_size), MATRIX),
                    s.up: TensorSpec((s.num_experts * s.intermediate_size, s.hidden_size), MATRIX),
                    s.down: TensorSpec((s.num_experts * s.hidden_size, s.intermediate_size), MATRIX)}

        def load(self, tensors, runtime):
            super().load(tensors, runtime)
            s = self.spec
            self.w = {name: runtime.matrix(tensors[getattr(s, name)]).float() for name in ("router", "gate", "up", "down")}

        def forward(self, ctx, x, residual):
            s, w = self.spec, self.w
            x = x.float()
            prob = torch.softmax(x @ w["router"].T, dim=-1)
            weight, expert = prob.max(dim=-1)
            F, d = s.intermediate_size, s.hidden_size
            for e in range(s.num_experts):
                h = torch.nn.functional.silu(x @ w["gate"][e * F:(e + 1) * F].T) * (x @ w["up"][e * F:(e + 1) * F].T)
                chosen = (weight * (expert == e))[:, None]
                residual += chosen * (h @ w["down"][e * d:(e + 1) * d].T)

    class DeviceDecayMixer(Part):
        """The decay mixer again, but a step of one token per sequence finds its rows of the state through
        ``ctx.slots`` on the device, so a captured graph of such a step serves any sequences."""
        capture_safe = True

        def __init__(self, spec):
            self.spec = spec

        def tensor_specs(self):
            return {self.spec.gain: TensorSpec((self.spec.hidden_size,), GAIN)}

        def load(self, tensors, runtime):
            super().load(tensors, runtime)
            self.gain = runtime.gain(tensors[self.spec.gain])

        def cache_request(self):
            return StateRequest((self.spec.hidden_size,), torch.float32)

        def forward(self, ctx, cache, x, residual):
            if ctx.all_single:
                slots = ctx.slots.long()
                state = cache.rows.index_select(0, slots) * self.spec.decay + x.float()
                cache.rows.index_copy_(0, slots, state)
                residual += state * self.gain
                return
            for seq in ctx.sequences:
                state = cache.rows[seq.slot]
                for t in range(seq.start, seq.start + seq.num_new):
                    state.mul_(self.spec.decay).add_(x[t].float())
                    residual[t] += state * self.gain

    return DistanceDecay, RoutedFeedForward, DeviceDecayMixer


def make_second_toy_config(state_mixer_kind):
    from llmplayer_b200.config.registry import ArchitectureConfig
    from llmplayer_b200.parts.specs import (
        AttentionSpec, BlockSpec, EmbeddingSpec, HeadSpec, ModelLayout, NormSpec, PositionSpec, SwiGLUSpec,
    )

    @dataclass(frozen=True)
    class SecondToyConfig(ArchitectureConfig):
        hidden_size: int
        vocab_size: int
        architecture = "SecondToyForTest"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["hidden_size"], raw["vocab_size"])

        def to_dict(self):
            return {"architectures": ["SecondToyForTest"], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size}

        def max_positions(self):
            return 512

        def layout(self):
            d = self.hidden_size
            attention = AttentionSpec(
                hidden_size=d, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
                position=PositionSpec("toy_distance", 16, 40, 0.8), q="l0.q", o="l0.o", k="l0.k", v="l0.v")
            mixer = (DeviceDecaySpec if state_mixer_kind == "toy_decay_device" else DecaySpec)(d, 0.9, "l1.gain")
            layers = (
                BlockSpec(NormSpec(d, 1e-5, "l0.n1"), attention, NormSpec(d, 1e-5, "l0.n2"),
                          RoutedSpec(d, 48, 3, "l0.router", "l0.g", "l0.u", "l0.d")),
                BlockSpec(NormSpec(d, 1e-5, "l1.n1"), mixer, NormSpec(d, 1e-5, "l1.n2"),
                          SwiGLUSpec(d, 64, "l1.g", "l1.u", "l1.d")),
            )
            return ModelLayout(EmbeddingSpec(self.vocab_size, d, "embed"), layers,
                               HeadSpec(self.vocab_size, d, NormSpec(d, 1e-5, "norm"), "head"))

    return SecondToyConfig


def plain_second_toy(w, tokens):
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)]
    # layer 0: attention with the distance-decay encoding, then the routed feed-forward
    h = P.rms_norm(x, w["l0.n1"], 1e-5)
    factor = torch.pow(torch.tensor(0.8, dtype=torch.float64), pos.double() / 40.0)[:, None, None]
    q = (h @ w["l0.q"].T).reshape(T, 4, 16) * factor
    k = (h @ w["l0.k"].T).reshape(T, 2, 16) / factor
    v = (h @ w["l0.v"].T).reshape(T, 2, 16)
    x = x + P.attention(q, k, v, 0.25, window=None, q_positions=pos).reshape(T, 64) @ w["l0.o"].T
    h = P.rms_norm(x, w["l0.n2"], 1e-5)
    prob = torch.softmax(h @ w["l0.router"].T, dim=-1)
    weight, expert = prob.max(dim=-1)
    out = torch.zeros_like(x)
    for t in range(T):
        e = int(expert[t])
        g, u, dn = w["l0.g"][e * 48:(e + 1) * 48], w["l0.u"][e * 48:(e + 1) * 48], w["l0.d"][e * 64:(e + 1) * 64]
        hid = torch.nn.functional.silu(h[t] @ g.T) * (h[t] @ u.T)
        out[t] = weight[t] * (hid @ dn.T)
    x = x + out
    # layer 1: the decay mixer, then a dense gated feed-forward
    h = P.rms_norm(x, w["l1.n1"], 1e-5)
    state = torch.zeros(64, dtype=torch.float64)
    mixed = torch.zeros_like(x)
    for t in range(T):
        state = 0.9 * state + h[t]
        mixed[t] = state * w["l1.gain"]
    x = x + mixed
    x = x + P.swiglu(P.rms_norm(x, w["l1.n2"], 1e-5), w["l1.g"], w["l1.u"], w["l1.d"])
    return P.rms_norm(x, w["norm"], 1e-5) @ w["head"].T


@pytest.mark.parametrize("state_mixer", ["toy_decay", "toy_decay_device"])
def test_other_positions_routing_and_graphs_over_other_slots(tmp_path, state_mixer):
    """A second toy architecture, registered from here: attention whose position encoding is no rotation (its
    part changes queries and keys itself, the kernels then run without rotation), a feed-forward with a router,
    and a state mixer. Decode steps of one batch are captured as CUDA graphs when every part reads the step
    from the device only (the device-indexed mixer); a later batch of the same shape that holds OTHER slots must
    still update its own rows of the state. With the host-indexed mixer the engine must not replay graphs at all."""
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import register_architecture, unregister_architecture
    from llmplayer_b200.parts import FEED_FORWARDS, MIXERS, POSITIONS
    from llmplayer_b200.weights import write_random_model
    distance, routed, device_decay = make_more_toys()
    POSITIONS.register("toy_distance", distance, replace=True)
    FEED_FORWARDS.register("toy_routed", routed, replace=True)
    MIXERS.register("toy_decay_device", device_decay, replace=True)
    MIXERS.register("toy_decay", make_decay_mixer(), replace=True)
    cfg = make_second_toy_config(state_mixer)
    register_architecture("SecondToyForTest", cfg, replace=True)
    try:
        model_dir = str(tmp_path / "toy2")
        write_random_model(cfg(hidden_size=64, vocab_size=89), 11, model_dir, dtype="bfloat16", std=0.1)
        weights = P.read_safetensors(os.path.join(model_dir, "model.safetensors"))
        eng = Engine.load(model_dir, dtype="bfloat16", max_tokens=8 * 128, max_slots=8)
        assert eng.model.capture_safe == (state_mixer == "toy_decay_device")
        seqs = [random_tokens(n, 89, seed=40 + n) for n in (30, 9, 70, 12, 33, 71)]
        refs = [plain_second_toy(weights, s) for s in seqs]

        def decode_together(group, slots, steps=6):
            """Prompts in one step, then `steps` tokens each; returns the decoded positions' logits per request."""
            fed = {i: len(seqs[i]) - steps for i in group}
            eng.step([(slots[i], seqs[i][:fed[i]]) for i in group], [[] for _ in group])
            rows = {i: [] for i in group}
            for _ in range(steps):
                out = eng.step([(slots[i], [seqs[i][fed[i]]]) for i in group], [[0] for _ in group]).cpu()
                for j, i in enumerate(group):
                    rows[i].append(out[j].clone())
                    fed[i] += 1
            return {i: torch.stack(rows[i]) for i in group}

        first = {i: eng.acquire() for i in (0, 1, 2)}                       # slots 0, 1, 2
        got = decode_together([0, 1, 2], first)
        if state_mixer == "toy_decay_device":
            assert any(g is not None for g, _ in eng._graphs.values()), "no decode step was captured"
        else:
            assert not eng._graphs
        parked = [eng.acquire() for _ in range(2)]                          # slots 3, 4 stay held
        for s in first.values():
            eng.release(s)
        second = {3: eng.acquire(), 4: eng.acquire(), 5: eng.acquire()}     # slots 0, 1, 2 again ...
        for s in list(second.values()):
            eng.release(s)
        more = [eng.acquire() for _ in range(3)]                            # ... kept away, so that the
        second = {i: eng.acquire() for i in (3, 4, 5)}                      # second batch holds slots 5, 6, 7
        assert sorted(second.values()) == [5, 6, 7]
        got.update(decode_together([3, 4, 5], second))
        for i, rows in got.items():
            assert_close(rows, refs[i][-6:], "bfloat16", f"second toy, request {i}", config="toy")
        for s in parked + more + list(second.values()):
            eng.release(s)
        assert eng.cache.slots.num_held == 0
    finally:
        unregister_architecture("SecondToyForTest")
        POSITIONS.unregister("toy_distance")
        FEED_FORWARDS.unregister("toy_routed")
        MIXERS.unregister("toy_decay_device")
        MIXERS.unregister("toy_decay")
