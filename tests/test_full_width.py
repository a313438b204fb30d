"""Two layers at the Llama-3.2-1B widths (2048 wide, 32 / 8 heads of 64, feed-forward 8192, vocabulary
128,256, llama3 rope scaling with factor 32) against the plain implementation in float64: each request
whole, the last 32 tokens one by one, and batches of twenty requests of unequal lengths whose shorter
ones end earlier and whose slots are used again. In float32 the engine must meet the plain logits to
2e-5 under every way of cutting the work; in bfloat16 these sizes put the kernels that tiny models never
reach under a model-level check: the persistent tcgen05 product (a request of more than 512 tokens), the
tcgen05 prompt attention, the 32-token decode tiles (twenty sequences), decode attention at 32 / 8 heads.

The plain implementation forms the head's logits only at the rows that are compared (its float64 head
over 128,256 entries is the slow part on the host)."""
import pytest
import torch

import plain_llama as P
from helpers import check_error, random_tokens, relative_error, tolerance

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                              "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
LENGTHS = [620, 150, 3, 64, 65, 129, 40, 17, 200, 1, 90, 33, 128, 70, 5, 111, 260, 48, 77, 96]


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    model_dir = str(tmp_path_factory.mktemp("wide") / "model")
    write_random_model(config_from_dict(WIDE), 2, model_dir, dtype="bfloat16")
    cfg, weights = P.read_model(model_dir)
    seqs = [random_tokens(n, 128256, seed=700 + i) for i, n in enumerate(LENGTHS)]
    return model_dir, cfg, weights, seqs


def rows_of_interest(n):
    """Positions of a sequence of n tokens that are compared: the first, the last, and both sides of page edges."""
    return sorted({p for p in (0, 1, 62, 63, 64, 65, 127, 128, 511, 512, n // 2, n - 2, n - 1) if 0 <= p < n})


class Checker:
    def __init__(self, cfg, weights, dtype):
        self.cfg, self.weights, self.dtype = cfg, weights, dtype
        self.worst = 0.0

    def check(self, tokens, rows, got, what):
        ref = P.forward(self.cfg, self.weights, tokens, dtype=torch.float64, rows=rows)
        err = check_error(f"1B-width logits, {self.dtype}", what, relative_error(got, ref), tolerance(self.dtype, "1B"))
        self.worst = max(self.worst, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_way_of_cutting_against_plain(wide, dtype, record_property):
    from llmplayer_b200 import Engine
    model_dir, cfg, weights, seqs = wide
    check = Checker(cfg, weights, dtype)
    need = sum(-(-n // 64) * 64 for n in LENGTHS)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=need, max_slots=len(seqs))

    # each request alone and whole (a handful of them: the long one, page edges, the shortest)
    for i in (0, 1, 3, 4, 5, 9):
        s, rows = seqs[i], rows_of_interest(len(seqs[i]))
        slot = eng.acquire()
        got = eng.step([(slot, s)], [rows]).cpu().clone()
        eng.release(slot)
        check.check(s, rows, got, f"whole, request {i}")

    # the last 32 tokens one by one
    for i in (0, 1, 4):
        s = seqs[i]
        head = max(1, len(s) - 32)
        slot = eng.acquire()
        first = eng.step([(slot, s[:head])], [[head - 1]]).cpu().clone()
        tail = [eng.step([(slot, [t])], [[0]]).cpu().clone() for t in s[head:]]
        eng.release(slot)
        rows = list(range(head - 1, len(s)))
        check.check(s, rows, torch.cat([first] + tail), f"last 32 one by one, request {i}")

    # twenty requests start together with half of their tokens, go on one token each; the shorter ones end
    # earlier; a second batch (the requests in another order) uses the slots and pages again
    for order in (list(range(20)), list(reversed(range(20)))):
        slots = {i: eng.acquire() for i in order}
        fed = {i: max(1, len(seqs[i]) // 2) for i in order}
        got = {i: {} for i in order}
        out = eng.step([(slots[i], seqs[i][:fed[i]]) for i in order], [[fed[i] - 1] for i in order]).cpu().clone()
        for j, i in enumerate(order):
            got[i][fed[i] - 1] = out[j]
        live = [i for i in order if fed[i] < len(seqs[i])]
        for i in order:
            if i not in live:
                eng.release(slots[i])
        while live:
            # logits are asked for at a request's first two and last two decoded tokens only
            want = [[0] if (fed[i] - max(1, len(seqs[i]) // 2) < 2 or len(seqs[i]) - fed[i] <= 2) else [] for i in live]
            out = eng.step([(slots[i], [seqs[i][fed[i]]]) for i in live], want).cpu().clone()
            at = 0
            for i, w in zip(live, want):
                if w:
                    got[i][fed[i]] = out[at]
                    at += 1
                fed[i] += 1
            for i in [i for i in live if fed[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if fed[i] < len(seqs[i])]
        eng.check()
        for i in order:
            rows = sorted(got[i])
            check.check(seqs[i], rows, torch.stack([got[i][r] for r in rows]), f"batch of twenty, request {i}")
        assert eng.cache.slots.num_held == 0
    record_property(f"worst_relative_error_{dtype}", check.worst)
    print(f"1B widths, {dtype}: worst relative error {check.worst:.3e}")
