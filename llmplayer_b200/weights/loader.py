"""Loading the tensors of a model folder by name, checked against the layout.

The reference fetches each tensor by its name and throws at the first missing
one (model/ModelLoader.java:695-701), without a shape check. Here the whole
folder is compared with what the model's parts expect, and one error lists
everything that is missing, unexpected or of the wrong shape.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import WeightError
from ..parts.specs import GAIN, INTEGER, MATRIX, TensorSpec
from .safetensors_io import open_model_files

_FLOATS = ("F32", "BF16", "F16", "F64")
_INTS = ("I32", "I64", "I16", "I8", "U8")


def held_dtype(stored: str, kind: str) -> torch.dtype:
    """The dtype a tensor is kept in: bfloat16 stays, anything stored in 32 bits
    (or in a format bfloat16 cannot hold exactly) is kept in float32, integer
    tables become int32."""
    if kind == INTEGER:
        return torch.int32
    return torch.bfloat16 if stored == "BF16" else torch.float32


def load_tensors(model_dir: str, expected: Mapping[str, TensorSpec]) -> Dict[str, torch.Tensor]:
    owners = open_model_files(model_dir)
    try:
        missing, wrong = [], []
        for name, spec in expected.items():
            if name not in owners:
                missing.append(name)
                continue
            dtype, shape = owners[name].info(name)
            if tuple(shape) != tuple(spec.shape):
                wrong.append(f"{name}: expected shape {list(spec.shape)}, file has {list(shape)}")
            elif spec.kind == INTEGER and dtype not in _INTS:
                wrong.append(f"{name}: expected an integer table, file has dtype {dtype}")
            elif spec.kind in (MATRIX, GAIN) and dtype not in _FLOATS:
                wrong.append(f"{name}: expected floating-point values, file has dtype {dtype}")
        unexpected = sorted(n for n in owners if n not in expected)
        if missing or wrong or unexpected:
            lines = [f"the tensors of {model_dir!r} do not fit the configuration:"]
            if missing:
                lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shape or type ({len(wrong)}):")
                lines.extend("    " + w for w in wrong)
            raise WeightError("\n".join(lines))
        out: Dict[str, torch.Tensor] = {}
        for name, spec in expected.items():
            handle = owners[name]
            stored, _ = handle.info(name)
            out[name] = handle.tensor(name).to(held_dtype(stored, spec.kind))
        return out
    finally:
        for handle in {id(h): h for h in owners.values()}.values():
            handle.close()
