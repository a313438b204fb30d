"""Interfaces of the parts and the registries that resolve a specification's kind.

A part is built from its specification alone, says which tensors it needs
(``tensor_specs``), takes them (``load``) and then works on the tensors of a
step. No part knows which model it is in.

* Norm:          ``apply(x[T, d] float32, out[T, d]) -> out`` (optionally on chosen rows)
* Position:      owned by a mixer: ``rotation()`` (a rule the kernels apply on the way) or
                 ``apply(ctx, qkv, ...)`` (any other rule, applied to the projection in place)
* Mixer:         ``cache_request()`` and ``forward(ctx, cache_view, x[T, d], residual[T, d])``:
                 adds its output into the float32 residual stream
* Feed-forward:  ``forward(ctx, x[T, d], residual[T, d])``: adds into the residual stream
* Block:         ``forward(ctx, cache_view, residual[T, d])``: one layer, in place

``ctx`` is the step's :class:`llmplayer_b200.engine.step.StepContext`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Optional

import torch

from ..errors import ConfigError
from .specs import TensorSpec


@dataclass
class Runtime:
    """Where and in which precision a model runs.

    ``dtype`` is ``"bfloat16"`` (activations and cache in bfloat16, tensor-core
    kernels) or ``"float32"`` (everything in true float32 through the plain
    kernels). ``kernels`` is ``"fast"`` or ``"plain"``: the latter forces the
    plain twins in bfloat16 too. The residual stream and the logits are float32
    in both.
    """
    device: torch.device
    dtype: str = "bfloat16"
    kernels: str = "fast"

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.kernels not in ("fast", "plain"):
            raise ConfigError(f"kernels must be 'fast' or 'plain', got {self.kernels!r}")

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.dtype == "bfloat16" else torch.float32

    @property
    def kv_dtype(self) -> torch.dtype:
        return self.act_dtype

    @property
    def fast(self) -> bool:
        return self.dtype == "bfloat16" and self.kernels == "fast"

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A weight matrix on the device: widened to float32 in the float32 path,
        kept as stored (bfloat16, or float32 if the file held 32 bits) otherwise.
        The same host tensor always yields the same device tensor, so a table that
        two parts name (a tied head) is held once."""
        memo = self.__dict__.setdefault("_uploaded", {})
        hit = memo.get(id(t))
        if hit is not None and hit[0] is t:
            return hit[1]
        if self.dtype == "float32":
            dev = t.to(device=self.device, dtype=torch.float32).contiguous()
        else:
            dev = t.to(device=self.device).contiguous()
        memo[id(t)] = (t, dev)
        return dev

    def shared(self, key, make):
        """One object per key for the whole model (parts of several layers that would otherwise each hold an
        equal table, such as rotary frequencies, hold the same one)."""
        memo = self.__dict__.setdefault("_shared", {})
        if key not in memo:
            memo[key] = make()
        return memo[key]

    def forget_uploads(self) -> None:
        """Drop the host tensors remembered by :meth:`matrix` (after a model is loaded)."""
        self.__dict__.pop("_uploaded", None)

    def gain(self, t: torch.Tensor) -> torch.Tensor:
        """A norm's gain: float32 always (widening is exact)."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()


@dataclass
class FollowingNorm:
    """A norm that comes right after a part's last product, offered to that part for fusion:
    if the part can make its product write ``norm(residual)`` to ``out`` (and zero ``clear``, a
    float32 buffer or None) on the way, it does so and says so by returning True."""
    norm: object
    out: torch.Tensor
    clear: Optional[torch.Tensor] = None


class PendingNorm:
    """``norm(source)`` that has not been computed yet: what a block hands to a part that declares
    ``takes_pending_norm = True`` instead of the normed tensor. Such a part may apply the norm inside
    its first product (it finds the float32 ``source`` and the ``norm`` part here); whenever it cannot,
    ``tensor()`` runs the norm as a kernel of its own (once) and returns the result."""

    def __init__(self, source: torch.Tensor, norm, materialize: Callable[[], torch.Tensor]):
        self.source = source
        self.norm = norm
        self._materialize = materialize
        self._tensor: Optional[torch.Tensor] = None

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self._materialize()
        return self._tensor

    @property
    def fusable(self) -> bool:
        return bool(getattr(self.norm, "fusable_rms", False))


class Part:
    # Steps of one token per sequence are replayed from CUDA graphs that were captured on an earlier step of
    # the same shape, possibly for other sequences. A part whose ``forward`` depends on the step only through
    # the device tensors of ``ctx`` (``tokens``, ``positions``, ``slots``, ``kv_len``, ``page_tables``...) and
    # through what the graph's key holds (batch, page-table widths, wanted rows) may say so; a part that reads
    # the step on the host (``ctx.sequences``, ``ctx.slot_list``: which rows of a state it updates, say)
    # leaves this False, and a model with such a part runs every step directly.
    capture_safe = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Callable] = {}

    def register(self, kind: str, factory: Callable, *, replace: bool = False) -> None:
        if kind in self._kinds and not replace and self._kinds[kind] is not factory:
            raise ConfigError(f"{self.what} kind {kind!r} is already registered")
        self._kinds[kind] = factory

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def build(self, spec):
        kind = getattr(spec, "kind", None)
        if kind not in self._kinds:
            raise ConfigError(f"unknown {self.what} kind {kind!r}; known: {', '.join(sorted(self._kinds))}")
        return self._kinds[kind](spec)

    def kinds(self):
        return tuple(sorted(self._kinds))


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
