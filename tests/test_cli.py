"""The command line: the reference's option names and defaults, and a run through the engine."""
import os
import subprocess
import sys

import pytest

from helpers import make_model
from llmplayer_b200.cli import CLIOptions, parse_ids

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_defaults_are_the_reference_ones():
    o = CLIOptions.parse(["model_dir"])
    assert o.model_path == "model_dir"                       # a bare first argument is the model
    assert (o.max_tokens, o.temperature, o.top_k, o.top_p, o.repetition_penalty) == (256, 0.7, 40, 0.9, 1.1)
    assert (o.min_p, o.mirostat, o.mirostat_tau, o.mirostat_eta) == (0.0, 0, 5.0, 0.1)
    assert (o.dry_multiplier, o.dry_base, o.dry_allowed_length, o.dry_range) == (0.0, 1.75, 2, 1024)
    assert o.context_length == 2048 and not o.interactive and not o.show_info
    c = o.to_sampler_config()
    assert (c.temperature, c.top_k, c.top_p, c.repetition_penalty) == (0.7, 40, 0.9, 1.1)


def test_flags_and_short_forms():
    o = CLIOptions.parse(["-m", "x", "-p", "1 2 3", "--prompt", "4,5", "-n", "7", "-t", "0", "--top-k", "5",
                          "--top-p", "0.5", "--repetition-penalty", "1.3", "--min-p", "0.05", "--mirostat", "2",
                          "--mirostat-tau", "3", "--mirostat-eta", "0.2", "--dry-multiplier", "0.8", "--dry-base", "2",
                          "--dry-allowed-length", "3", "--dry-range", "64", "--seed", "9", "-c", "128", "--threads", "4",
                          "--gpu", "--gpu-layers", "3", "--stop-ids", "7,8", "--bogus"])
    assert o.model_path == "x" and [parse_ids(p) for p in o.prompts] == [[1, 2, 3], [4, 5]]
    assert (o.max_tokens, o.temperature, o.top_k, o.top_p, o.seed, o.context_length) == (7, 0.0, 5, 0.5, 9, 128)
    assert o.stop_ids == [7, 8] and o.unknown == ["--bogus"]
    c = o.to_sampler_config()
    assert c.is_greedy and c.mirostat == 2 and c.dry_range == 64 and c.seed == 9 and c.min_p == 0.05


def test_help_runs_without_a_gpu():
    out = subprocess.run([sys.executable, "-m", "llmplayer_b200", "--help"], cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 0 and "--max-tokens, -n" in out.stdout and "--repetition-penalty" in out.stdout


@pytest.mark.gpu
def test_cli_generates_and_prints_the_stats_line(tmp_path):
    model_dir = make_model(tmp_path, "A", dtype="bfloat16")
    cmd = [sys.executable, "-m", "llmplayer_b200", "-m", model_dir, "-p", "5 17 3", "-p", "9 1", "-n", "5", "-t", "0",
           "--repetition-penalty", "1.0", "-c", "64"]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    assert "--- Generation ---" in lines and "--- Stats ---" in lines
    assert lines[-1].startswith("Tokens: 5 prompt + 10 generated in ") and lines[-1].endswith("tok/s)")
    rows = [l for l in lines if l.startswith("[0] ") or l.startswith("[1] ")]
    assert len(rows) == 2 and all(len(r.split()) == 6 for r in rows)
    info = subprocess.run([sys.executable, "-m", "llmplayer_b200", model_dir, "--info"], cwd=ROOT, capture_output=True,
                          text=True, timeout=300)
    assert info.returncode == 0 and "LlamaForCausalLM" in info.stdout and "num_hidden_layers" in info.stdout
