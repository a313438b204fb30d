#!/usr/bin/env python3
"""Benchmark: decode tokens per second of the Llama-3.2-1B shape with random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch. The default run has a batch of 8
sequences with 512-token prompts in a cache sized for a context of 4096. It prints ONE
JSON line: ``value`` = decoded tokens per second timed on the device with CUDA events
(K steps back to back), ``e2e`` = the same through ``Engine.generate`` with host tokens
in and out, ``prefill`` = one 2,048-token prompt, ``roofline`` = bytes a decode step must
read over its time against the HBM peak, ``points`` = decode at batch 1 and 64.
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

# Llama-3.2-1B sizes (the benchmark configuration), as config.json keys
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    "torch_dtype": "bfloat16",
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

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
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 6:
                continue
            try:
                sm.append(float(row[0]))
                mx.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(names, row[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_bytes(cfg, layers, batch, context, engine):
    """Bytes one decode step has to read: every weight it uses once and the cache of the live requests."""
    d, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (H * hd * d + 2 * G * hd * d + d * H * hd + 3 * d * F) * 2
    weights = layers * per_layer + V * d * 2
    cache = batch * context * layers * 2 * G * hd * 2
    return weights + cache


def prefill_flops(cfg, layers, T):
    d, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, G, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = layers * (H * hd * d + 2 * G * hd * d + d * H * hd + 3 * d * F)
    attention = layers * 2 * H * hd * T * T          # causal: half of 4 H hd T^2
    return 2.0 * linear * T + attention + 2.0 * V * d


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (both are reported)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points and the prefill")
    ap.add_argument("--prefill-only", action="store_true",
                    help="measure only the 2,048-token prefill (small runs for profiling)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "DenzoSOFTHub/LLMPlayer is a Java/Maven project: pip finds neither setup.py nor "
                          "pyproject.toml, and this image has no JVM to run it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU library")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from llmplayer_b200 import Engine
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.engine.decode import DecodeSession
    from llmplayer_b200.kernels import ops
    from llmplayer_b200.sampling import SamplerConfig
    from llmplayer_b200.weights import write_random_model

    peaks = load_peaks()
    cfg = dict(LLAMA_1B)
    model_layers = cfg["num_hidden_layers"]
    layers = args.layers or model_layers
    cfg["num_hidden_layers"] = layers
    tmp = tempfile.mkdtemp(prefix="llmplayer_b200_bench_")
    try:
        write_random_model(config_from_dict(cfg), 2, tmp, dtype="bfloat16")
        max_batch = 1 if args.prefill_only else max(args.batch, 1 if args.no_points else 64)
        engine = Engine.load(tmp, dtype="bfloat16", context_length=args.context, max_batch=max_batch)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    gen = torch.Generator().manual_seed(2)

    def prompts(batch, length):
        return torch.randint(0, cfg["vocab_size"], (batch, length), generator=gen).tolist()

    def timed_decode(batch, steps, warmup, sample_clocks=False):
        """K decode steps back to back on the device, greedy feedback, timed with CUDA events."""
        session = DecodeSession(engine, prompts(batch, args.prompt_len), reserve=args.prompt_len + steps + warmup + 1)
        try:
            session.run(warmup)
            torch.cuda.synchronize()
            clocks = ClockSampler() if sample_clocks else None
            if clocks:
                clocks.start()
                time.sleep(0.3)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches_before = ops.launch_count()
            torch.cuda.synchronize()
            start.record()
            session.run(steps)
            stop.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(stop)
            launches = session.launches_per_step * steps if session.launches_per_step else \
                ops.launch_count() - launches_before
            context = args.prompt_len + warmup + steps // 2
            return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                    "context": context, "clocks": clocks.stop() if clocks else None}
        finally:
            session.close()

    def timed_prefill(T=2048):
        slot = engine.acquire()
        ptoks = prompts(1, T)[0]
        for _ in range(2):                       # warm-up passes over the same slot
            engine.step([(slot, ptoks)], [[T - 1]])
            engine.release(slot)
            slot = engine.acquire()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([(slot, ptoks)], [[T - 1]])
        stop.record()
        torch.cuda.synchronize()
        engine.release(slot)
        ms = start.elapsed_time(stop)
        flops = prefill_flops(cfg, layers, T)
        return {"value": T / (ms / 1e3), "tokens": T, "ms": ms,
                "frac": flops / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "of": peaks["source"]}

    if args.prefill_only:
        print(json.dumps({"metric": "prefill tok/s (Llama-3.2-1B shape, bf16)", "impl": "ours", "layers": layers,
                          "model_layers": model_layers, "prefill": timed_prefill()}))
        return 0

    main_run = timed_decode(args.batch, args.steps, args.warmup, sample_clocks=True)
    bytes_step = decode_bytes(cfg, layers, args.batch, main_run["context"], engine)
    achieved = bytes_step / (main_run["ms_per_step"] / 1e3) / 1e9

    # end to end through the Python entry point: host token ids in, host token ids out
    e2e_prompts = prompts(args.batch, args.prompt_len)
    engine.generate(e2e_prompts, SamplerConfig.greedy(), max_tokens=args.warmup, stop_token_ids=())
    engine.generate(e2e_prompts, SamplerConfig.greedy(), max_tokens=args.steps, stop_token_ids=())
    st = engine.last_generation_stats
    e2e = {"value": st.decode_tokens_per_second, "unit": "tokens/s",
           "h2d_bytes_per_step": engine.last_step_h2d_bytes + engine._sampler.last_h2d_bytes,
           "d2h_bytes_per_step": engine._sampler.last_d2h_bytes}

    result = {
        "metric": "decode tok/s (Llama-3.2-1B shape, bf16, batch %d)" % args.batch,
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0, 0.02) and uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B shape", "layers": layers, "model_layers": model_layers, "hidden_size": 2048,
            "heads": 32, "kv_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
            "global_batch": args.batch, "seq_len": args.context, "prompt_len": args.prompt_len,
            "decode_context_mid": main_run["context"], "parallelism": "single GPU",
            "l2": "inputs larger than L2 (a step reads %.2f GB)" % (bytes_step / 1e9),
            "peaks": peaks["source"],
        },
        "clocks": main_run["clocks"],
        "e2e": e2e,
        "gpu_launches": int(main_run["launches"]),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "of": peaks["source"]},
    }
    if not args.no_points:
        result["prefill"] = timed_prefill()
        points = {}
        for b in (1, 64):
            steps = max(16, args.steps // 2)
            points[f"decode_b{b}"] = timed_decode(b, steps, max(3, args.warmup // 2))["tok_s"]
        # the same entry point with the reference's default sampler (temperature 0.7, top-k 40, top-p 0.9,
        # repetition penalty 1.1) instead of the greedy choice
        engine.generate(e2e_prompts, SamplerConfig(seed=1), max_tokens=max(3, args.warmup // 2), stop_token_ids=())
        engine.generate(e2e_prompts, SamplerConfig(seed=1), max_tokens=max(16, args.steps // 2), stop_token_ids=())
        points["e2e_reference_sampler"] = engine.last_generation_stats.decode_tokens_per_second
        result["points"] = points
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
