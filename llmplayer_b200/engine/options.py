"""The engine's options as one typed object.

The reference spreads the same choices over its command-line object
(cli/CLIOptions.java:71-201: context length, device, sampler defaults) and JVM
system properties read where they are used (``cuda.nograph``, ``cuda.profile``,
``cuda.cublas``...: java21 inference/CudaForwardPass.java:430-431, :790, :1142).
Here they are fields of :class:`EngineOptions`, passed to ``Engine.load``;
the command line mirrors them as flags, and the kernel switches have
environment variables of the same meaning for runs that cannot pass options.
"""
from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class EngineOptions:
    # precision and kernels
    dtype: str = "bfloat16"              # "bfloat16" or "float32" (everything in true 32-bit)
    kernels: str = "fast"                # "plain": the plain twins of every kernel, in bfloat16 too
    # sizes
    context_length: Optional[int] = None  # per sequence; default and upper bound: the model's own limit
    beyond_model_context: bool = False   # let context_length exceed the model's max_position_embeddings
    max_batch: int = 1                   # with context_length, sizes the cache when max_tokens is not given
    max_tokens: Optional[int] = None     # positions the cache holds in all
    max_slots: Optional[int] = None      # sequences held at once (default: as many as there are pages)
    device: str = "cuda:0"
    # how steps run
    graphs: bool = True                  # replay captured CUDA graphs for steps of one token per sequence
    host_loop: bool = True               # greedy decoding runs several steps per call of the native host loop
    profile: bool = False                # time each section of the model walk with CUDA events (no graphs)
    # kernel switches (None: leave the process-wide setting, which starts from the environment)
    pdl: Optional[bool] = None
    few_tokens: Optional[int] = None
    fewtok_kernel: Optional[bool] = None
    ring_shared: Optional[int] = None
    ring_alone: Optional[int] = None
    ring_alone_tile: Optional[int] = None
    ring_normed: Optional[int] = None

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.kernels not in ("fast", "plain"):
            raise ConfigError(f"kernels must be 'fast' or 'plain', got {self.kernels!r}")
        for name in ("context_length", "max_tokens", "max_slots"):
            value = getattr(self, name)
            if value is not None and int(value) <= 0:
                raise ConfigError(f"{name} must be positive, got {value}")
        if int(self.max_batch) <= 0:
            raise ConfigError(f"max_batch must be positive, got {self.max_batch}")

    def kernel_settings(self) -> dict:
        return {name: getattr(self, name) for name in ("pdl", "few_tokens", "fewtok_kernel", "ring_shared", "ring_alone",
                                                          "ring_alone_tile", "ring_normed")
                if getattr(self, name) is not None}

    def with_changes(self, **changes) -> "EngineOptions":
        known = {f.name for f in fields(self)}
        unknown = sorted(set(changes) - known)
        if unknown:
            raise ConfigError(f"unknown engine option(s): {', '.join(unknown)}; known: {', '.join(sorted(known))}")
        return replace(self, **changes)
