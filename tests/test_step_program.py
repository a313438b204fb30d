"""The persistent step kernel (a decode step as one launch): its logits against the plain
implementation, for batches of unequal lengths, heads of 64 and of 128, and sizes that are no
power of two; and that a model with a part that cannot emit keeps running as a chain of kernels."""
import os

import pytest
import torch

from helpers import assert_close, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

PROGRAM_A = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 320, "vocab_size": 1000, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 512,
}
PROGRAM_B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 264, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 712, "vocab_size": 1303, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 1024,
}


def _model(tmp_path, raw, seed, std):
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.weights import write_random_model
    out = os.path.join(str(tmp_path), f"program_{raw['hidden_size']}")
    write_random_model(config_from_dict(raw), seed, out, dtype="bfloat16", std=std)
    return out


@pytest.mark.parametrize("raw,batch,std", [(PROGRAM_A, 1, 0.05), (PROGRAM_A, 5, 0.05), (PROGRAM_B, 8, 0.04),
                                           (PROGRAM_B, 16, 0.04)])
def test_program_steps_match_plain(tmp_path, raw, batch, std):
    from llmplayer_b200 import Engine
    from llmplayer_b200.kernels import ops
    model_dir = _model(tmp_path, raw, 3, std)
    eng = Engine.load(model_dir, dtype="bfloat16", context_length=512, max_batch=batch)
    eng.model.use_program = True
    lengths = [3 + (37 * i) % 140 for i in range(batch)]           # unequal; some cross a page boundary while decoding
    lengths[0] = 62
    steps = 6
    seqs = [random_tokens(n + steps, raw["vocab_size"], 10 + i) for i, n in enumerate(lengths)]
    slots = [eng.acquire() for _ in range(batch)]
    eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, lengths)], [[] for _ in range(batch)])
    got = [[] for _ in range(batch)]
    for k in range(steps):
        logits = eng.step([(s, [q[n + k]]) for s, q, n in zip(slots, seqs, lengths)], [[0]] * batch)
        for i in range(batch):
            got[i].append(logits[i].float().cpu().clone())
    ops.check_kernel_status()
    programs = [p for p in eng.model._programs.values() if p is not None]
    assert programs, "the step did not run as a program"
    for i in range(batch):
        ref = plain_logits(model_dir, seqs[i])[lengths[i]:]
        assert_close(torch.stack(got[i]), ref, "bfloat16", f"sequence {i}")
    eng.close()


def test_wanted_rows_are_a_subset(tmp_path):
    """A step that wants the logits of some sequences only."""
    from llmplayer_b200 import Engine
    model_dir = _model(tmp_path, PROGRAM_A, 4, 0.05)
    eng = Engine.load(model_dir, dtype="bfloat16", context_length=256, max_batch=3)
    eng.model.use_program = True
    seqs = [random_tokens(n, 1000, 20 + i) for i, n in enumerate((9, 70, 33))]
    slots = [eng.acquire() for _ in seqs]
    eng.step([(s, q[:-1]) for s, q in zip(slots, seqs)], [[], [], []])
    logits = eng.step([(s, [q[-1]]) for s, q in zip(slots, seqs)], [[0], [], [0]]).float().cpu()
    assert logits.shape[0] == 2
    assert [p for p in eng.model._programs.values() if p is not None]
    assert_close(logits[0], plain_logits(model_dir, seqs[0])[-1], "bfloat16", "first")
    assert_close(logits[1], plain_logits(model_dir, seqs[2])[-1], "bfloat16", "third")
    eng.close()


def test_model_without_emit_runs_as_kernels(tmp_path):
    """Head sizes the program has no unit for: the step is refused as a program and runs as before."""
    from helpers import make_model
    from llmplayer_b200 import Engine
    model_dir = make_model(tmp_path, "C")                          # heads of 48
    eng = Engine.load(model_dir, dtype="bfloat16", context_length=128, max_batch=2)
    eng.model.use_program = True
    seq = random_tokens(20, 301, 5)
    slot = eng.acquire()
    eng.step([(slot, seq[:-1])], [[]])
    logits = eng.step([(slot, [seq[-1]])], [[0]]).float().cpu()
    assert all(p is None for p in eng.model._programs.values())
    assert_close(logits[0], plain_logits(model_dir, seq)[-1], "bfloat16")
    eng.close()
