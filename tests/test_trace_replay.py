"""bin/trace_run, driven as a user drives it: the same requests whole, with the last
32 tokens one by one, and in batches of unequal lengths whose slots are used again."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TINY, assert_close, make_model, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def run_trace(model_dir, dtype, steps, out_dir, max_tokens):
    """Feed the steps one at a time, waiting for each ``done`` line as the protocol asks."""
    proc = subprocess.Popen(
        [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(max_tokens)],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for step in steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {step['step']}", line
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


def read_logits(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())


def requests_for(name, lengths):
    vocab = TINY[name][0]["vocab_size"]
    return {f"r{i}": random_tokens(n, vocab, seed=100 + i) for i, n in enumerate(lengths)}


def collect(out_dir, steps, vocab):
    """Logits per request id and position, gathered from the step files."""
    got = {}
    pos = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        if not wanted:
            continue
        rows = read_logits(out_dir, step["step"], vocab)
        assert rows.shape[0] == wanted
        r = 0
        for e in step["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = rows[r]
                r += 1
        for e in step["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
    return got


def check_all(got, reqs, model_dir, dtype, what, config):
    for rid, toks in reqs.items():
        ref = plain_logits(model_dir, toks)
        have = torch.stack([got[rid][p] for p in range(len(toks))])
        assert_close(have, ref, dtype, f"{what} request {rid}", config=config)


def steps_whole(reqs):
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(reqs.items())]


def steps_tail(reqs, tail=32):
    steps = []
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def steps_batches(reqs, batch, prompt_frac=0.5):
    """Batches of ``batch`` requests that start together with a prefix of each request,
    then go on by one token each; shorter requests end earlier; batches follow one another."""
    steps = []
    ids = list(reqs)
    for b0 in range(0, len(ids), batch):
        group = ids[b0:b0 + batch]
        fed = {}
        entries = []
        for rid in group:
            n = max(1, int(len(reqs[rid]) * prompt_frac))
            entries.append({"id": rid, "tokens": reqs[rid][:n], "want": list(range(n))})
            fed[rid] = n
        done = [rid for rid in group if fed[rid] == len(reqs[rid])]
        steps.append({"step": len(steps), "entries": entries, "end": done})
        live = [rid for rid in group if rid not in done]
        while live:
            entries = [{"id": rid, "tokens": [reqs[rid][fed[rid]]], "want": [0]} for rid in live]
            for rid in live:
                fed[rid] += 1
            done = [rid for rid in live if fed[rid] == len(reqs[rid])]
            steps.append({"step": len(steps), "entries": entries, "end": done})
            live = [rid for rid in live if rid not in done]
    return steps


# tiny-D has heads of 64: its prompts of more than 64 tokens take the tcgen05 prompt attention, the request of
# 600 tokens spans ten pages, and batches of 20 decode with the products' 32-token tiles
CASES = [("A", [5, 9, 13, 40, 70], 3), ("B", [1, 7, 16, 30, 65, 129], 3),
         ("D", [600, 130, 70, 33, 200, 66, 129, 90] + [3 + 5 * i for i in range(32)], 20)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,batch", CASES)
def test_replay_whole_tail_batches(tmp_path, name, lengths, batch, dtype):
    model_dir = make_model(tmp_path, name, dtype=dtype)
    vocab = TINY[name][0]["vocab_size"]
    reqs = requests_for(name, lengths)
    longest = -(-max(lengths) // 64) * 64
    by_need = sorted((-(-n // 64) * 64 for n in lengths), reverse=True)
    for what, steps, max_tokens in [
        ("whole", steps_whole(reqs), longest),
        ("tail32", steps_tail(reqs), longest),
        # `batch` requests at a time: the cache is sized for the largest batch only, so slots
        # and pages of finished requests must be used again by the next batch
        ("batches", steps_batches(reqs, batch), sum(by_need[:batch])),
    ]:
        out_dir = str(tmp_path / f"{what}_{dtype}")
        run_trace(model_dir, dtype, steps, out_dir, max_tokens)
        check_all(collect(out_dir, steps, vocab), reqs, model_dir, dtype, f"tiny-{name} {what}", name)


def test_replay_without_wanted_rows_writes_no_file(tmp_path):
    model_dir = make_model(tmp_path, "A", dtype="float32")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": [4], "want": [0]}], "end": ["x"]}]
    out_dir = str(tmp_path / "out")
    run_trace(model_dir, "float32", steps, out_dir, 64)
    assert not os.path.exists(os.path.join(out_dir, "0.f32"))
    got = read_logits(out_dir, 1, 256)
    assert_close(got, plain_logits(model_dir, [1, 2, 3, 4])[-1:], "float32", "after an unwatched step")
