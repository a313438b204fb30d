"""A linear map held as an [out, in] matrix, and the choice of the kernel that applies it.

Reference: tensor/FloatTensor.java:49-67 (row-major [rows, cols], one dot product per
output row) and the per-dtype kernels src/main/resources/kernels/cuda/matmul_f32.cu,
matmul_bf16.cu.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops
from .base import Runtime


class Linear:
    """out (=|+=) x @ W^T for W = the given matrices stacked by rows; ``gated=True`` takes a
    (gate, up) pair and offers the gated product silu(x gate^T) * (x up^T)."""

    def __init__(self, parts: Sequence[torch.Tensor], runtime: Runtime, gated: bool = False):
        mats = [runtime.matrix(p) for p in parts]
        if len({m.dtype for m in mats}) > 1:        # mixed storage: widen to the widest
            mats = [m.to(torch.float32) for m in mats]
        self.runtime = runtime
        self.gated = gated
        self.in_features = mats[0].shape[1]
        self.out_features = sum(m.shape[0] for m in mats)
        self.interleaved = False
        if gated:
            if len(mats) != 2 or mats[0].shape != mats[1].shape:
                raise ValueError("a gated product takes a gate and an up matrix of equal shape")
            self.out_features = mats[0].shape[0]
            self.interleaved = runtime.fast and mats[0].dtype == torch.bfloat16 and self.in_features % 8 == 0
        if self.interleaved:
            # the tensor-core kernel wants gate and up rows of the same features side by side
            self.weight = ops.interleave_gate_up(mats[0], mats[1])
        else:
            self.weight = mats[0] if len(mats) == 1 else torch.cat(mats, dim=0).contiguous()

    def _fast(self) -> bool:
        # the tensor-core kernel wants bfloat16 operands and rows of a multiple of 8 elements (TMA strides)
        return self.runtime.fast and self.weight.dtype == torch.bfloat16 and self.in_features % 8 == 0

    def tensor_cores(self) -> bool:
        """Whether this map's products run on the tensor-core kernels (bfloat16 weights, rows of a multiple of 8)."""
        return self._fast()

    def store(self, x: torch.Tensor, out: torch.Tensor, ctx=None) -> torch.Tensor:
        return self._run(x, out, ops.STORE, ctx)

    def accumulate(self, x: torch.Tensor, out: torch.Tensor, ctx=None, then_norm=None) -> bool:
        """out += x @ W^T. ``then_norm`` (a :class:`FollowingNorm`): if this product runs on the
        tensor cores for a few rows and the norm is an RMS norm over whole rows, the product's
        last CTA also writes the norm; returns whether it did."""
        if (then_norm is not None and ctx is not None and self._fast() and x.dtype == torch.bfloat16
                and x.shape[0] <= ops.FUSED_NORM_MAX_TOKENS and getattr(then_norm.norm, "fusable_rms", False)
                and then_norm.out.dtype == torch.bfloat16 and out.shape[1] == self.out_features
                and self.out_features % 128 == 0):
            ctx.take_cleared()
            norm = then_norm.norm
            ops.gemm(x, self.weight, out, ops.ACCUMULATE,
                     norm_after=(norm.weight, norm.spec.eps, then_norm.out, then_norm.clear,
                                 ctx.counters("product_ctas", 1)))
            return True
        self._run(x, out, ops.ACCUMULATE, ctx)
        return False

    def swiglu(self, x: torch.Tensor, out: torch.Tensor, ctx=None) -> torch.Tensor:
        return self._run(x, out, ops.SWIGLU, ctx)

    def sums_into(self, ctx, tokens: int, out_name: str, mode: int):
        """The float32 buffer that this product, run for ``tokens`` rows, will add partial
        sums into and that must therefore be zero beforehand; None if it stores its result.
        ``out_name``: the workspace name of its output."""
        if not self._fast() or mode != ops.STORE:
            return None
        _, splits = ops.gemm_plan(tokens, self.out_features, self.in_features, mode)
        if splits <= 1:
            return None
        return ctx.buffer(out_name, (tokens, self.out_features), torch.float32)

    def can_few(self, tokens: int, mode: int) -> bool:
        """Whether :meth:`few` serves this product for ``tokens`` rows."""
        return self._fast() and tokens <= ops.FEW_TOKENS and (mode != ops.SWIGLU or self.interleaved)

    def few(self, x: torch.Tensor, out: torch.Tensor, mode: int, *, norm=None, sumsq=None, zero=None) -> bool:
        """The product for a handful of rows with what a decode step fuses around it (see
        :func:`ops.gemm_few`); ``norm``: an RMS norm part applied to the float32 ``x`` on the way in.
        Returns whether ``out`` still lacks the rows' factors (then ``sumsq`` holds their sums of squares)."""
        return ops.gemm_few(x, self.weight, out, mode, norm=None if norm is None else (norm.weight, norm.spec.eps),
                            sumsq=sumsq, zero=zero)

    def _run(self, x, out, mode, ctx):
        if self._fast() and x.dtype == torch.bfloat16 and (mode != ops.SWIGLU or self.interleaved):
            cleared = ctx.take_cleared() if ctx is not None else False
            return ops.gemm(x, self.weight, out, mode, cleared=cleared)
        return ops.gemm_plain(x, self.weight, out, mode)
