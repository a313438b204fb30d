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
    assert_close(logits, plain_logits(model_dir, tokens), dtype, f"tiny-{name} whole", config=name)


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
    assert_close(got[:4], ref[:4], dtype, "first tokens", config="C")
    assert_close(got, ref, dtype, "long decoding", config="C")


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


def test_full_width_layers_bfloat16_against_float32(tmp_path):
    """Two layers at the Llama-3.2-1B widths (2048 wide, 32/8 heads of 64, 8192, vocabulary 128256, llama3
    rope scaling): the bfloat16 engine (tensor-core products and attention at their real sizes, prompt and
    decode kernels) against the float32 engine, whole and then token by token."""
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    raw = {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
        "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                                  "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    }
    model_dir = str(tmp_path / "wide")
    write_random_model(config_from_dict(raw), 2, model_dir, dtype="bfloat16")
    tokens = random_tokens(333, 128256, seed=4)
    want = [0, 100, 199, 200, 332]
    logits = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.load(model_dir, dtype=dtype, max_tokens=512)
        slot = eng.acquire()
        whole = eng.step([(slot, tokens)], [want]).cpu().clone()
        eng.release(slot)
        slot = eng.acquire()
        eng.step([(slot, tokens[:200])], [[]])
        tail = [eng.step([(slot, [t])], [[0]]).cpu().clone() for t in tokens[200:]]
        eng.release(slot)
        logits[dtype] = (whole, torch.cat([tail[0], tail[-1]]))
        eng.close()
        del eng
        torch.cuda.empty_cache()
    ref_whole, ref_tail = logits["float32"]
    assert torch.equal(ref_whole[3:], ref_tail)                       # float32: cutting into steps changes nothing
    assert_close(logits["bfloat16"][0], ref_whole, "bfloat16", "1B widths, whole", config="1B")
    assert_close(logits["bfloat16"][1], ref_tail, "bfloat16", "1B widths, decoded", config="1B")


@pytest.mark.parametrize("batch", [12, 20, 40])
def test_full_width_decode_batches(tmp_path, batch):
    """Sequences of unequal lengths decoding together at the Llama-3.2-1B widths, against the float32 engine.
    Twelve: the tcgen05 products with operand makers for the two products behind a norm (the row factor of q|k|v
    left to the attention kernel), the few-token products with two tiles of 8 tokens for the other two. Twenty:
    tcgen05 products with a 32-token tile throughout. Forty: 64-token tiles and norm kernels of their own."""
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    raw = {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
        "rope_theta": 500000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
        "max_position_embeddings": 4096,
    }
    model_dir = str(tmp_path / "wide12")
    write_random_model(config_from_dict(raw), 7, model_dir, dtype="bfloat16")
    lengths = [5 + 11 * (i % 12) + i // 12 for i in range(batch)]    # 5 .. 126: some cross a page boundary
    steps = 3
    seqs = [random_tokens(n + steps, 128256, seed=30 + i) for i, n in enumerate(lengths)]
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.load(model_dir, dtype=dtype, max_tokens=batch * 192, max_slots=batch)
        slots = [eng.acquire() for _ in seqs]
        eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, lengths)], [[] for _ in seqs])
        outs = []
        for k in range(steps):
            outs.append(eng.step([(s, [q[n + k]]) for s, q, n in zip(slots, seqs, lengths)], [[0]] * batch).cpu().clone())
        eng.check()
        got[dtype] = torch.stack(outs)
        eng.close()
        del eng
        torch.cuda.empty_cache()
    assert_close(got["bfloat16"], got["float32"], "bfloat16", f"1B widths, {batch} sequences", config="1B")


def test_wider_layers_with_heads_of_128(tmp_path):
    """Two layers at the widths of a larger model of the family (4096 wide, 32/8 heads of 128, 14336, an odd
    vocabulary, untied head): prompts of unequal lengths in one step, then three decode steps of the batch of
    eight, bfloat16 against float32."""
    from helpers import relative_error
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    raw = {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 32003,
        "rope_theta": 500000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
        "max_position_embeddings": 8192,
    }
    model_dir = str(tmp_path / "wider")
    write_random_model(config_from_dict(raw), 3, model_dir, dtype="bfloat16")
    lengths = [700, 40, 333, 64, 65, 129, 1, 512]
    steps = 3
    seqs = [random_tokens(n + steps, 32003, seed=50 + i) for i, n in enumerate(lengths)]
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.load(model_dir, dtype=dtype, max_tokens=8 * 768, max_slots=8)
        slots = [eng.acquire() for _ in seqs]
        outs = [eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, lengths)], [[n - 1] for n in lengths]).cpu().clone()]
        for k in range(steps):
            outs.append(eng.step([(s, [q[n + k]]) for s, q, n in zip(slots, seqs, lengths)], [[0]] * 8).cpu().clone())
        eng.check()
        got[dtype] = torch.stack(outs)
        eng.close()
        del eng
        torch.cuda.empty_cache()
    for k in range(steps + 1):
        assert_close(got["bfloat16"][k], got["float32"][k], "bfloat16", f"wider layers, step {k}", config="wider")


@pytest.mark.parametrize("stored,dtype", [("float32", "bfloat16"), ("bfloat16", "float32")])
def test_stored_and_compute_dtypes_may_differ(tmp_path, stored, dtype):
    """A folder stored in 32 bits run in bfloat16 keeps its float32 matrices (plain products with
    bfloat16 activations); a bfloat16 folder run in float32 is widened exactly."""
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, "B", dtype=stored)
    tokens = random_tokens(70, TINY["B"][0]["vocab_size"], seed=2)
    eng = Engine.load(model_dir, dtype=dtype, max_tokens=128)
    if dtype == "bfloat16":
        assert eng.model.blocks[0].mixer.qkv.weight.dtype == torch.float32        # stored in 32 bits: stays so
    slot = eng.acquire()
    got = [eng.step([(slot, tokens[:40])], [list(range(40))]).cpu().clone()]
    got += [eng.step([(slot, [t])], [[0]]).cpu().clone() for t in tokens[40:]]
    eng.release(slot)
    assert_close(torch.cat(got), plain_logits(model_dir, tokens), dtype, f"{stored} folder in {dtype}", config="B")
