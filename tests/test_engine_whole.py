"""Each request alone and whole, against the plain implementation."""
import pytest
import torch

from helpers import TINY, assert_close, make_model, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,length", [("A", 13), ("B", 30), ("B", 1), ("C", 200)])
def test_whole_sequence(tmp_path, name, length, dtype):
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, name, dtype="float32" if dtype == "float32" else "bfloat16")
    tokens = random_tokens(length, TINY[name][0]["vocab_size"], seed=length)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=512)
    slot = eng.acquire()
    logits = eng.step([(slot, tokens)], [list(range(length))]).cpu()
    eng.release(slot)
    assert_close(logits, plain_logits(model_dir, tokens), dtype, f"tiny-{name} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tmp_path, dtype):
    """A one-token prompt, then 330 tokens one by one (five page boundaries); every position's
    logits, the very first ones included, against the whole-sequence plain implementation."""
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, "C", dtype=dtype)
    tokens = random_tokens(331, TINY["C"][0]["vocab_size"], seed=9)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=384)
    slot = eng.acquire()
    rows = [eng.step([(slot, [t])], [[0]]).cpu().clone() for t in tokens]
    eng.release(slot)
    got = torch.cat(rows)
    ref = plain_logits(model_dir, tokens)
    assert_close(got[:4], ref[:4], dtype, "first tokens")
    assert_close(got, ref, dtype, "long decoding")


def test_steps_are_checked(tmp_path):
    from llmplayer_b200 import Engine
    from llmplayer_b200.errors import CacheError, CacheFull, RequestError
    model_dir = make_model(tmp_path, "A", dtype="float32")
    eng = Engine.load(model_dir, dtype="float32", max_tokens=128, context_length=100)
    slot = eng.acquire()
    with pytest.raises(RequestError, match="vocabulary"):
        eng.step([(slot, [1, 256])], [[0]])
    with pytest.raises(RequestError, match="wanted place"):
        eng.step([(slot, [1, 2])], [[2]])
    with pytest.raises(RequestError, match="at least one token"):
        eng.step([(slot, [])], [[]])
    with pytest.raises(RequestError, match="context length"):
        eng.step([(slot, [1] * 101)], [[]])
    with pytest.raises(CacheError):
        eng.step([(slot + 1, [1])], [[0]])
    other = eng.acquire()
    eng.step([(slot, [1] * 65)], [[]])                       # two pages: the cache of 128 positions is now full
    with pytest.raises(CacheFull):
        eng.step([(other, [1])], [[0]])
    eng.release(slot)
    assert eng.step([(other, [1])], [[0]]).shape == (1, 256)
