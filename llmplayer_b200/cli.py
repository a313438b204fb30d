"""Command line, with the reference's option names and meanings where it has them.

Reference: cli/CLIOptions.java:71-201 (flags), :260-324 (usage text),
cli/CLIRunner.java:113-143 (single prompt: generate, then the line
``Tokens: P prompt + G generated in T ms (R tok/s)``), :187-224 (interactive loop).
There is no tokenizer here: a prompt is a list of token ids ("1 15 7" or "1,15,7").
"""
from __future__ import annotations

import sys
import time
from typing import List, Optional

USAGE = """Usage: python -m llmplayer_b200 [options]

Options:
  --model, -m <dir>        Model folder (config.json + model.safetensors)
  --prompt, -p <ids>       Prompt as token ids, e.g. "1 15 7" (repeat for a batch)
  --prompt-file <path>     One prompt of token ids per line (a batch)
  --interactive, -i        Read one prompt (token ids) per line from standard input
  --max-tokens, -n <num>   Max tokens to generate (default: 256)
  --temperature, -t <num>  Sampling temperature, 0 = greedy (default: 0.7)
  --top-k <num>            Top-K sampling (default: 40)
  --top-p <num>            Top-P nucleus sampling (default: 0.9)
  --repetition-penalty <n> Repetition penalty (default: 1.1)
  --min-p <num>            min-P sampling (default: 0 = off)
  --mirostat <0|2>         Mirostat sampler: 0=off, 2=mirostat v2 (default: 0)
  --mirostat-tau <num>     Mirostat target entropy (default: 5.0)
  --mirostat-eta <num>     Mirostat learning rate (default: 0.1)
  --dry-multiplier <num>   DRY sampler multiplier (default: 0 = off)
  --dry-base <num>         DRY exponential base (default: 1.75)
  --dry-allowed-length <n> DRY min match length (default: 2)
  --dry-range <num>        DRY lookback window (default: 1024)
  --seed <num>             Random seed
  --context-length, -c <n> Max context length (default: 2048)
  --stop-ids <ids>         Token ids that end a sequence (default: the model's eos_token_id)
  --dtype <name>           bfloat16 (default) or float32
  --max-slots <num>        Sequences held at once (default: one per prompt)
  --no-graph               Run every step directly instead of replaying captured CUDA graphs
  --profile                Time each section of the model walk (disables graphs) and print ms per step
  --plain-kernels          Use the plain twin of every kernel
  --gpu-device <id>        CUDA device index (default: 0)
  --random <seed>          Write random weights for the config.json in --model first
  --info                   Show model info and exit
  --help, -h               Show this help
"""


class CLIOptions:
    def __init__(self):
        self.model_path: Optional[str] = None
        self.prompts: List[str] = []
        self.interactive = False
        self.max_tokens = 256
        self.temperature = 0.7
        self.top_k = 40
        self.top_p = 0.9
        self.repetition_penalty = 1.1
        self.seed: Optional[int] = None
        self.min_p = 0.0
        self.mirostat = 0
        self.mirostat_tau = 5.0
        self.mirostat_eta = 0.1
        self.dry_multiplier = 0.0
        self.dry_base = 1.75
        self.dry_allowed_length = 2
        self.dry_range = 1024
        self.context_length = 2048
        self.stop_ids: Optional[List[int]] = None
        self.dtype = "bfloat16"
        self.gpu_device = 0
        self.random_seed: Optional[int] = None
        self.prompt_file: Optional[str] = None
        self.max_slots: Optional[int] = None
        self.no_graph = False
        self.profile = False
        self.plain_kernels = False
        self.show_info = False
        self.help = False
        self.unknown: List[str] = []

    _VALUE_FLAGS = {
        "--model": ("model_path", str), "-m": ("model_path", str),
        "--max-tokens": ("max_tokens", int), "-n": ("max_tokens", int),
        "--temperature": ("temperature", float), "-t": ("temperature", float),
        "--top-k": ("top_k", int), "--top-p": ("top_p", float),
        "--repetition-penalty": ("repetition_penalty", float), "--min-p": ("min_p", float),
        "--mirostat": ("mirostat", int), "--mirostat-tau": ("mirostat_tau", float),
        "--mirostat-eta": ("mirostat_eta", float), "--dry-multiplier": ("dry_multiplier", float),
        "--dry-base": ("dry_base", float), "--dry-allowed-length": ("dry_allowed_length", int),
        "--dry-range": ("dry_range", int), "--seed": ("seed", int),
        "--context-length": ("context_length", int), "-c": ("context_length", int),
        "--dtype": ("dtype", str), "--gpu-device": ("gpu_device", int), "--random": ("random_seed", int),
        "--prompt-file": ("prompt_file", str), "--max-slots": ("max_slots", int),
    }
    _SWITCHES = {"--no-graph": "no_graph", "--profile": "profile", "--plain-kernels": "plain_kernels"}
    # flags of the reference that place work on devices or threads; accepted, without effect here
    _IGNORED_WITH_VALUE = ("--threads", "--gpu-layers", "--gpu-backend", "--gpu-memory")
    _IGNORED = ("--gpu", "--gpu-chain", "--no-gpu-chain")

    @classmethod
    def parse(cls, args: List[str]) -> "CLIOptions":
        o = cls()
        i = 0
        while i < len(args):
            a = args[i]
            if a in cls._VALUE_FLAGS:
                name, kind = cls._VALUE_FLAGS[a]
                i += 1
                if i >= len(args):
                    raise SystemExit(f"option {a} needs a value")
                setattr(o, name, kind(args[i]))
            elif a in ("--prompt", "-p"):
                i += 1
                o.prompts.append(args[i])
            elif a == "--stop-ids":
                i += 1
                o.stop_ids = parse_ids(args[i])
            elif a in cls._SWITCHES:
                setattr(o, cls._SWITCHES[a], True)
            elif a in ("--interactive", "-i"):
                o.interactive = True
            elif a == "--info":
                o.show_info = True
            elif a in ("--help", "-h"):
                o.help = True
            elif a in cls._IGNORED_WITH_VALUE:
                i += 1
            elif a in cls._IGNORED:
                pass
            elif a == "--no-gpu":
                raise SystemExit("--no-gpu: this library runs on the GPU only")
            elif o.model_path is None and not a.startswith("-"):
                o.model_path = a            # a bare first argument is the model path
            else:
                print(f"Unknown option: {a}", file=sys.stderr)
                o.unknown.append(a)
            i += 1
        return o

    def to_engine_options(self, batch: int):
        """The engine's options that this command line asks for (engine/options.py)."""
        from .engine.options import EngineOptions
        return EngineOptions(
            dtype=self.dtype, kernels="plain" if self.plain_kernels else "fast", context_length=self.context_length,
            max_batch=batch, max_slots=self.max_slots, device=f"cuda:{self.gpu_device}", graphs=not self.no_graph,
            profile=self.profile)

    def to_sampler_config(self):
        from .sampling.params import SamplerConfig
        kwargs = dict(
            temperature=self.temperature, top_k=self.top_k, top_p=self.top_p,
            repetition_penalty=self.repetition_penalty, min_p=self.min_p, mirostat=self.mirostat,
            mirostat_tau=self.mirostat_tau, mirostat_eta=self.mirostat_eta, dry_multiplier=self.dry_multiplier,
            dry_base=self.dry_base, dry_allowed_length=self.dry_allowed_length, dry_range=self.dry_range)
        if self.seed is not None:
            kwargs["seed"] = self.seed
        return SamplerConfig(**kwargs)


def parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def _print_result(index: int, total: int, response) -> None:
    if response.error:
        print(response.error)
        return
    head = f"[{index}] " if total > 1 else ""
    print(head + " ".join(str(t) for t in response.token_ids))


def run(argv: Optional[List[str]] = None) -> int:
    opts = CLIOptions.parse(list(sys.argv[1:] if argv is None else argv))
    if opts.help or opts.model_path is None:
        print(USAGE)
        return 0 if opts.help else 2
    if opts.random_seed is not None:
        from .config import load_config
        from .weights import write_random_model
        write_random_model(load_config(opts.model_path), opts.random_seed, opts.model_path, dtype=opts.dtype)
    from .engine import Engine
    prompts = [parse_ids(p) for p in opts.prompts]
    if opts.prompt_file is not None:
        with open(opts.prompt_file) as fh:
            prompts += [parse_ids(line) for line in fh if line.strip()]
    batch = max(1, len(prompts))
    engine = Engine.load(opts.model_path, opts.to_engine_options(batch))
    if opts.show_info:
        print(engine.info())
        return 0

    def generate(prompts: List[List[int]]) -> None:
        print("\n--- Generation ---")
        start = time.perf_counter()
        responses = engine.generate(prompts, opts.to_sampler_config(), max_tokens=opts.max_tokens,
                                    stop_token_ids=opts.stop_ids)
        elapsed_ms = (time.perf_counter() - start) * 1e3
        for i, r in enumerate(responses):
            _print_result(i, len(responses), r)
        stats = engine.last_generation_stats
        print("--- Stats ---")
        print("Tokens: %d prompt + %d generated in %dms (%.1f tok/s)" % (
            sum(r.prompt_token_count for r in responses), sum(r.token_count for r in responses),
            elapsed_ms, stats.decode_tokens_per_second))
        if opts.profile:
            # as the reference's -Dcuda.profile=true prints: milliseconds per section (java21
            # inference/CudaForwardPass.java:1431-1456)
            report = engine.profile_report(reset=True)
            print("--- Profile (%d steps, ms per step) ---" % report["steps"])
            for name, row in report["sections"].items():
                print("  %-20s %8.3f  (%d calls)" % (name, row["ms_per_step"], row["calls"]))

    if prompts:
        generate(prompts)
    if opts.interactive:
        print("Interactive mode: one prompt of token ids per line, 'quit' to leave.")
        for line in sys.stdin:
            line = line.strip()
            if line in ("quit", "exit"):
                break
            if line:
                generate([parse_ids(line)])
    elif not prompts:
        print("No prompt given: use --prompt or --interactive.", file=sys.stderr)
        return 2
    return 0
