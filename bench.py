#!/usr/bin/env python3
"""Benchmark: decode tokens per second of a Llama shape with random bf16 weights, through ``Engine.generate``.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 1b|3b|8b]

One "step" is one decode step of the whole batch. The default run has the Llama-3.2-1B shape, a batch of 8
sequences with 512-token prompts in a cache sized for a context of 4096. Every figure comes from the library's
own generation loop (host token ids in, host token ids out): one generation call per measured point, whose first W
decode steps are warm-up and whose following decode steps are timed in laps of exactly K steps; the median over
the laps is reported. It prints ONE JSON line:

* ``value``: decoded tokens per second of a lap of K steps on the device's clock (CUDA events at the lap's
  boundaries), ``e2e``: the same laps on the host's clock;
* ``prefill``: one 2,048-token prompt; ``roofline``: the bytes a decode step must read over its time against
  the HBM peak; ``points``: decode at batch 1 and 64, and at contexts of about 1,024 / 2,048 / 3,584 for
  batches of 1, 8 and 64, with ``points_detail`` giving ms per step, bytes and the HBM fraction of each.

``--shape 3b`` / ``8b`` run the other two shapes the baseline names (batch 16 with prompts of 64 to 1,024 tokens
and 256 steps; batch 32 with 2,048-token prompts and 512 steps) unless ``--steps`` says otherwise.
``--profile`` adds the device time per section of the model walk (a separate, short run in profile mode).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def llama_shape(layers, hidden, heads, kv_heads, head_dim, ffn, factor, tied):
    return {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": layers, "hidden_size": hidden,
        "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": ffn, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": tied, "max_position_embeddings": 131072,
        "torch_dtype": "bfloat16",
    }


# name -> (config.json keys, seed, batch, prompt lengths (lo, hi), decode steps, context the cache is sized for)
SHAPES = {
    "1b": ("Llama-3.2-1B shape", llama_shape(16, 2048, 32, 8, 64, 8192, 32.0, True), 2, 8, (512, 512), 256, 4096),
    "3b": ("Llama-3.2-3B shape", llama_shape(28, 3072, 24, 8, 128, 8192, 32.0, True), 3, 16, (64, 1024), 256, 1280),
    "8b": ("Llama-3.1-8B shape", llama_shape(32, 4096, 32, 8, 128, 14336, 8.0, False), 4, 32, (2048, 2048), 512, 2560),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
REPEATS = 5


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            raw = json.load(fh)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                "source": "measured"}
    except (OSError, ValueError, KeyError):
        return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi for the whole run; a window of the samples
    (by wall-clock time) is summarised for each measured point."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def window(self, begin, end):
        sm, mx, reasons = [], [], set()
        for stamp, row in list(self.rows):
            if not begin - 0.05 <= stamp <= end + 0.15 or len(row) < 6:
                continue
            try:
                sm.append(float(row[0]))
                mx.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(self.NAMES, row[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def layer_weights(cfg):
    d, F = cfg["hidden_size"], cfg["intermediate_size"]
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    return H * hd * d + 2 * G * hd * d + d * H * hd + 3 * d * F


def decode_bytes(cfg, layers, cached_tokens):
    """Bytes one decode step has to read: every weight it uses once (the layers and the head; of the embedding
    only the gathered rows, which are not counted) and the keys and values of the live requests."""
    G, hd = cfg["num_key_value_heads"], cfg["head_dim"]
    weights = (layers * layer_weights(cfg) + cfg["vocab_size"] * cfg["hidden_size"]) * 2
    return weights + cached_tokens * layers * 2 * G * hd * 2


def prefill_flops(cfg, layers, lengths):
    H, hd = cfg["num_attention_heads"], cfg["head_dim"]
    tokens = sum(lengths)
    attention = layers * sum(2 * H * hd * n * n for n in lengths)          # causal: half of 4 H hd n^2
    return 2.0 * layers * layer_weights(cfg) * tokens + attention + 2.0 * cfg["vocab_size"] * cfg["hidden_size"] * len(lengths)


def spread(values):
    return {"median": statistics.median(values), "min": min(values), "max": max(values), "repeats": len(values)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES))
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both are reported)")
    ap.add_argument("--repeats", type=int, default=REPEATS)
    ap.add_argument("--no-points", action="store_true", help="skip the other batches and contexts and the prefill")
    ap.add_argument("--prefill-only", action="store_true",
                    help="measure only the 2,048-token prefill (small runs for profiling)")
    ap.add_argument("--profile", action="store_true", help="add the device time per section of the model walk")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "DenzoSOFTHub/LLMPlayer is a Java/Maven project: pip finds neither setup.py nor "
                          "pyproject.toml, and this image has no JVM to run it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU library")
        return 2
    args.warmup = max(3, args.warmup)
    repeats = max(1, args.repeats)

    import torch
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.sampling import SamplerConfig
    from llmplayer_b200.weights import write_random_model

    peaks = load_peaks()
    title, base, seed, batch0, (len_lo, len_hi), steps0, context0 = SHAPES[args.shape]
    cfg = dict(base)
    model_layers = cfg["num_hidden_layers"]
    layers = args.layers or model_layers
    cfg["num_hidden_layers"] = layers
    batch = args.batch or batch0
    steps = args.steps or steps0
    if args.prompt_len:
        len_lo = len_hi = args.prompt_len
    context = args.context or max(context0, len_hi + args.warmup + repeats * steps + 2)
    main_shape = args.shape == "1b"
    with_points = main_shape and not args.no_points and not args.prefill_only
    tmp = tempfile.mkdtemp(prefix="llmplayer_b200_bench_")
    try:
        write_random_model(config_from_dict(cfg), seed, tmp, dtype="bfloat16")
        max_batch = 1 if args.prefill_only else max(batch, 64 if with_points else 1)
        engine = Engine.load(tmp, dtype="bfloat16", context_length=context, max_batch=max_batch)
        profiled = Engine.load(tmp, dtype="bfloat16", context_length=context, max_batch=batch, profile=True) \
            if args.profile else None
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    gen = torch.Generator().manual_seed(seed)
    clocks = ClockSampler()
    clocks.start()

    def prompts(count, lo, hi):
        lengths = [lo] * count if lo == hi else torch.randint(lo, hi + 1, (count,), generator=gen).tolist()
        return [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]

    greedy = SamplerConfig.greedy()

    def timed_decode(count, lo, hi, k, warmup, sampler=greedy):
        """One generation call through Engine.generate: the prompts, `warmup` untimed decode steps, then
        `repeats` laps of exactly k decode steps each, timed on the device (CUDA events at the lap boundaries) and
        on the host; the medians over the laps are reported."""
        ps = prompts(count, lo, hi)
        begin = time.time()
        engine.generate(ps, sampler, max_tokens=warmup + repeats * k + 1, stop_token_ids=(), laps=(warmup, k))
        end = time.time()
        laps = engine.last_generation_stats.laps
        assert len(laps) == repeats and all(lap["steps"] == k and lap["tokens"] == count * k for lap in laps), laps
        device = [lap["tokens"] / (lap["device_ms"] / 1e3) for lap in laps]
        host = [lap["tokens"] / (lap["host_ms"] / 1e3) for lap in laps]
        tok_s = statistics.median(device)
        ms = count / tok_s * 1e3
        cached = sum(len(p) for p in ps) + count * (warmup + repeats * k // 2)      # the live requests' cache, mid-run
        nbytes = decode_bytes(cfg, layers, cached)
        return {"tok_s": tok_s, "ms_per_step": ms, "e2e_tok_s": statistics.median(host),
                "launches": int(statistics.median(lap.get("launches", 0) for lap in laps)),
                "context_mid": cached // count, "gb_per_step": nbytes / 1e9,
                "hbm_frac": nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
                "spread_tok_s": spread(device), "clocks": clocks.window(begin, end),
                "h2d": engine.last_step_h2d_bytes, "d2h": engine.last_step_d2h_bytes}

    def timed_prefill(lengths):
        ps = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
        times = []
        for i in range(2 + repeats):                  # two warm-up passes
            slots = [engine.acquire() for _ in ps]
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step(list(zip(slots, ps)), [[len(p) - 1] for p in ps])
            stop.record()
            torch.cuda.synchronize()
            for s in slots:
                engine.release(s)
            if i >= 2:
                times.append(start.elapsed_time(stop))
        ms = statistics.median(times)
        tokens = sum(lengths)
        return {"value": tokens / (ms / 1e3), "tokens": tokens, "ms": ms,
                "frac": prefill_flops(cfg, layers, lengths) / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12),
                "of": peaks["source"], "spread_ms": spread(times)}

    try:
        if args.prefill_only:
            print(json.dumps({"metric": f"prefill tok/s ({title}, bf16)", "impl": "ours", "layers": layers,
                              "model_layers": model_layers, "prefill": timed_prefill([2048])}))
            return 0

        run = timed_decode(batch, len_lo, len_hi, steps, args.warmup)
        result = {
            "metric": "decode tok/s (%s, bf16, batch %d)" % (title, batch),
            "value": run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
            "ms_per_step": run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: seeded random weights N(0, 0.02) and uniform random token ids",
            "impl": "ours",
            "config": {
                "model": title, "layers": layers, "model_layers": model_layers, "hidden_size": cfg["hidden_size"],
                "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"],
                "vocab_size": cfg["vocab_size"], "global_batch": batch, "seq_len": context,
                "prompt_len": len_lo if len_lo == len_hi else f"{len_lo}-{len_hi}",
                "decode_context_mid": run["context_mid"], "parallelism": "single GPU",
                "l2": "inputs larger than L2 (a step reads %.2f GB)" % run["gb_per_step"],
                "peaks": peaks["source"], "repeats": repeats, "timed": "median over laps of K decode steps inside one "
                "Engine.generate call, CUDA events",
            },
            "clocks": run["clocks"],
            "e2e": {"value": run["e2e_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": run["h2d"],
                    "d2h_bytes_per_step": run["d2h"]},
            "gpu_launches": int(run["launches"]),
            "roofline": {"bound": "hbm", "achieved": run["hbm_frac"] * peaks["hbm_gbs"], "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": run["hbm_frac"], "of": peaks["source"]},
            "spread": run["spread_tok_s"],
        }
        if not main_shape and not args.no_points:
            # the other shapes: the prompts of the run itself, processed in one step
            lengths = [len(p) for p in prompts(batch, len_lo, len_hi)]
            result["prefill"] = timed_prefill(lengths)
        if with_points:
            result["prefill"] = timed_prefill([2048])
            points, detail = {}, {}

            def point(name, count, length, k, sampler=greedy):
                r = timed_decode(count, length, length, k, max(3, args.warmup // 2), sampler)
                points[name] = r["tok_s"]
                detail[name] = {key: r[key] for key in ("ms_per_step", "gb_per_step", "hbm_frac", "context_mid",
                                                        "e2e_tok_s", "spread_tok_s", "clocks")}
            k = max(16, steps // 2)
            for b in (1, 64):
                point(f"decode_b{b}", b, len_lo, k)
            warm = max(3, args.warmup // 2)
            for length in (1024, 2048, 3584):
                for b in (1, 8, 64):
                    # prompts such that the middle of the timed steps lies at this context, within the cache's 4096
                    kk = max(1, min(k, (2 * (context - 1 - length) - warm) // repeats))
                    point(f"decode_b{b}_ctx{length}", b, length - (warm + repeats * kk) // 2, kk)
            # the same entry point with the reference's default sampler (temperature 0.7, top-k 40, top-p 0.9,
            # repetition penalty 1.1) instead of the greedy choice: every step goes through the interpreter
            r = timed_decode(batch, len_lo, len_hi, k, max(3, args.warmup // 2), SamplerConfig(seed=1))
            points["e2e_reference_sampler"] = r["e2e_tok_s"]
            result["points"] = points
            result["points_detail"] = detail
        if profiled is not None:
            ps = prompts(batch, len_lo, len_hi)
            profiled.generate(ps, greedy, max_tokens=4, stop_token_ids=())
            profiled.profile_report(reset=True)
            profiled.generate(ps, greedy, max_tokens=1, stop_token_ids=())
            prefill_sections = profiled.profile_report(reset=True)
            profiled.generate(ps, greedy, max_tokens=min(steps, 32) + 1, stop_token_ids=())
            report = profiled.profile_report()
            result["profile"] = {"decode_and_prompt": report, "prompt_only": prefill_sections,
                                 "note": "sections timed with CUDA events in profile mode (no graphs, no overlap "
                                         "between kernels); the second entry is one call that stops after the prompt"}
        print(json.dumps(result))
        return 0
    finally:
        clocks.stop()


if __name__ == "__main__":
    sys.exit(main())
