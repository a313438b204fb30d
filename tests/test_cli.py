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


def test_engine_switches_become_engine_options(tmp_path):
    o = CLIOptions.parse(["-m", "x", "--prompt-file", "p.txt", "--max-slots", "5", "--no-graph", "--profile",
                          "--plain-kernels", "--dtype", "float32", "-c", "300", "--gpu-device", "1"])
    assert o.prompt_file == "p.txt" and o.max_slots == 5 and o.no_graph and o.profile and o.plain_kernels
    e = o.to_engine_options(batch=3)
    assert (e.dtype, e.kernels, e.context_length, e.max_batch, e.max_slots) == ("float32", "plain", 300, 3, 5)
    assert e.device == "cuda:1" and e.graphs is False and e.profile is True
    d = CLIOptions.parse(["x"]).to_engine_options(batch=1)
    assert d.graphs and not d.profile and d.kernels == "fast" and d.max_slots is None


def test_engine_options_are_checked():
    from llmplayer_b200.engine.options import EngineOptions
    from llmplayer_b200.errors import ConfigError
    with pytest.raises(ConfigError, match="dtype"):
        EngineOptions(dtype="float16")
    with pytest.raises(ConfigError, match="max_tokens"):
        EngineOptions(max_tokens=0)
    with pytest.raises(ConfigError, match="unknown engine option.*warp_speed"):
        EngineOptions().with_changes(warp_speed=9)
    o = EngineOptions().with_changes(few_tokens=8, pdl=False)
    assert o.kernel_settings() == {"few_tokens": 8, "pdl": False}


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
    # prompts from a file, sections timed: the profile lines follow the stats line
    prompt_file = tmp_path / "prompts.txt"
    prompt_file.write_text("5 17 3\n\n9,1\n")
    prof = subprocess.run([sys.executable, "-m", "llmplayer_b200", "-m", model_dir, "--prompt-file", str(prompt_file),
                           "-n", "4", "-t", "0", "--repetition-penalty", "1.0", "-c", "64", "--profile"],
                          cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert prof.returncode == 0, prof.stderr
    assert "Tokens: 5 prompt + 8 generated in " in prof.stdout
    tail = prof.stdout.split("--- Profile (")[1]
    assert tail.startswith("4 steps") and "attention.scores" in tail and "ffn.gate_up" in tail and "head.proj" in tail
    info = subprocess.run([sys.executable, "-m", "llmplayer_b200", model_dir, "--info"], cwd=ROOT, capture_output=True,
                          text=True, timeout=300)
    assert info.returncode == 0 and "LlamaForCausalLM" in info.stdout and "num_hidden_layers" in info.stdout
