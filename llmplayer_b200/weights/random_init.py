"""Seeded random weights, written as a model folder.

The reference has no such mode (it needs a GGUF file); tests and benchmarks
here need models of any size without a download. Every matrix is drawn from
N(0, std), every norm gain from 1 + N(0, std), in float32 from one seeded
generator, tensor after tensor in the order the layout names them; the result
is then stored in the requested dtype.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping

import torch

from ..config.registry import ArchitectureConfig
from ..errors import WeightError
from ..parts.specs import GAIN, INTEGER, MATRIX, TensorSpec
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, std: float = 0.02,
                   dtype: str = "bfloat16") -> Dict[str, torch.Tensor]:
    if dtype not in _STORE:
        raise WeightError(f"random weights can be stored as {sorted(_STORE)}, not {dtype!r}")
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if spec.kind == INTEGER:
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
            continue
        draw = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std
        if spec.kind == GAIN:
            draw += 1.0
        elif spec.kind != MATRIX:
            raise WeightError(f"tensor {name!r}: unknown kind {spec.kind!r}")
        out[name] = draw.to(_STORE[dtype])
    return out


def write_random_model(config: ArchitectureConfig, seed: int, out_dir: str, *, dtype: str = "bfloat16",
                       std: float = 0.02) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``out_dir``."""
    from ..engine.model import expected_tensors  # parts are needed to know the tensors

    os.makedirs(out_dir, exist_ok=True)
    tensors = random_tensors(expected_tensors(config.layout()), seed, std=std, dtype=dtype)
    raw = config.to_dict()
    raw["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(raw, fh, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    return out_dir
