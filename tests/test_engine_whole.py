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
