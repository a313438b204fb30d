"""Tiny configurations and comparison helpers shared by the tests."""
import os

import torch

import plain_llama

# Two tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 320, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
}
# A third one for long sequences: heads wider than the width / heads, odd sizes.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 176, "vocab_size": 301, "rope_theta": 25000.0,
    "rope_scaling": None, "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 1024,
}
# A fourth one with heads of 64, the size the tcgen05 prompt attention is built for (head count x head size
# differs from the width), for prompts of hundreds of tokens and batches of more than sixteen sequences.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 272, "vocab_size": 515, "rope_theta": 100000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "rms_norm_eps": 2e-5, "tie_word_embeddings": True, "max_position_embeddings": 2048,
}
TINY = {"A": (TINY_A, 0, 0.02), "B": (TINY_B, 1, 0.05), "C": (TINY_C, 5, 0.08), "D": (TINY_D, 8, 0.06)}

# Largest |engine - plain| allowed, as a fraction of the largest |plain| logit. float32: 2e-5 everywhere. bfloat16:
# the error grows with a model's depth and widths, so each configuration has its own bound, set to at most four
# times the worst error that the comparisons of that configuration achieved on a B200 (tiny-A 1.8e-3, tiny-B 6.7e-3,
# tiny-C 6.3e-3, tiny-D 9.0e-3, the toy architecture 5.2e-3, two layers at the Llama-3.2-1B widths 9.2e-3, two
# layers 4096 / 14336 wide 1.2e-2); the session prints the achieved errors at its end (conftest.py).
TOLERANCE = {"float32": 2e-5, "bfloat16": 4e-2}
BFLOAT16_BOUND = {"A": 7e-3, "B": 2.5e-2, "C": 2.5e-2, "D": 3.5e-2, "toy": 2e-2, "1B": 3.5e-2, "wider": 4e-2}


def tolerance(dtype, config=None):
    if dtype == "float32":
        return TOLERANCE["float32"]
    return BFLOAT16_BOUND.get(config, TOLERANCE["bfloat16"])


def make_model(tmp_path, name, dtype="bfloat16"):
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    raw, seed, std = TINY[name]
    out = os.path.join(str(tmp_path), f"tiny{name}_{dtype}")
    write_random_model(config_from_dict(raw), seed, out, dtype=dtype, std=std)
    return out


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(model_dir, tokens, rows=None):
    cfg, w = plain_llama.read_model(model_dir)
    return plain_llama.forward(cfg, w, tokens, dtype=torch.float64, rows=rows)


# Every comparison of the engine with a reference leaves its achieved error here; the session prints the worst
# per kind at its end and writes all of them to $LLMPLAYER_B200_ERROR_LOG (a JSON file) when that is set.
ACHIEVED = []


def record_error(kind, what, err, bound):
    ACHIEVED.append({"kind": kind, "what": what, "error": float(err), "bound": float(bound)})


def check_error(kind, what, err, bound):
    """Record an achieved error and hold it against its bound."""
    record_error(kind, what, err, bound)
    assert err <= bound, f"{what}: error {err:.3e} exceeds {bound:.1e} ({kind})"
    return err


def relative_error(got, ref):
    got = torch.as_tensor(got, dtype=torch.float64).cpu()
    ref = torch.as_tensor(ref, dtype=torch.float64).cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), "engine produced non-finite logits"
    return float((got - ref).abs().max() / ref.abs().max())


def assert_close(got, ref, dtype, what="", config=None):
    """``config``: which configuration's bfloat16 bound applies (a key of ``BFLOAT16_BOUND``)."""
    return check_error(f"model logits, {dtype}", what, relative_error(got, ref), tolerance(dtype, config))
