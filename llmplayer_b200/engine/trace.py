"""Trace replay: given token ids in, logits out, through the engine's own step function.

The reference has no such program; its nearest relatives print predictions while
stepping through a prompt (DiagnosticRunner.java:323-340) and return logits for
given tokens (api/LLMEngine.java:941-1033).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--context-length", type=int, default=None,
                    help="longest request; default: the model's max_position_embeddings. A larger value is taken "
                         "as given (positions beyond what the model was made for)")
    args = ap.parse_args(argv)

    from .engine import Engine

    os.makedirs(args.out, exist_ok=True)
    engine = Engine.load(args.model, dtype=args.dtype, max_tokens=max(args.max_tokens, 64), device=args.device,
                         context_length=args.context_length, beyond_model_context=args.context_length is not None)
    slots: Dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries, want = [], []
        for entry in step.get("entries", []):
            rid = str(entry["id"])
            if rid not in slots:
                slots[rid] = engine.acquire()
            entries.append((slots[rid], entry["tokens"]))
            want.append(entry.get("want", []))
        if entries:
            logits = engine.step(entries, want)
            engine.check()                     # a kernel that gave up waiting must not pass as a result
            if logits.shape[0]:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                path = os.path.join(args.out, f"{step['step']}.f32")
                with open(path + ".tmp", "wb") as fh:
                    fh.write(np.ascontiguousarray(arr).tobytes())
                os.replace(path + ".tmp", path)
        for rid in step.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.release(slots.pop(rid))
        print(f"done {step['step']}", flush=True)
    return 0
