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
    """out (=|+=) x @ W^T, or the gated product when W stacks gate rows over up rows."""

    def __init__(self, parts: Sequence[torch.Tensor], runtime: Runtime):
        mats = [runtime.matrix(p) for p in parts]
        if len({m.dtype for m in mats}) > 1:        # mixed storage: widen to the widest
            mats = [m.to(torch.float32) for m in mats]
        self.weight = mats[0] if len(mats) == 1 else torch.cat(mats, dim=0).contiguous()
        self.runtime = runtime
        self.out_features, self.in_features = self.weight.shape

    def _fast(self) -> bool:
        # the tensor-core kernel wants bfloat16 operands and rows of a multiple of 8 elements (TMA strides)
        return (self.runtime.fast and self.weight.dtype == torch.bfloat16 and self.in_features % 8 == 0
                and ops.fast_gemm_available())

    def store(self, x: torch.Tensor, out: torch.Tensor, ctx=None) -> torch.Tensor:
        return self._run(x, out, ops.STORE, ctx)

    def accumulate(self, x: torch.Tensor, out: torch.Tensor, ctx=None) -> torch.Tensor:
        return self._run(x, out, ops.ACCUMULATE, ctx)

    def swiglu(self, x: torch.Tensor, out: torch.Tensor, ctx=None) -> torch.Tensor:
        return self._run(x, out, ops.SWIGLU, ctx)

    def sums_into(self, ctx, tokens: int, out_name: str, mode: int):
        """The float32 buffer that this product, run for ``tokens`` rows, will add partial
        sums into and that must therefore be zero beforehand; None if it stores its result.
        ``out_name``: the workspace name of its output."""
        if not self._fast() or mode == ops.ACCUMULATE:
            return None
        features = self.out_features // 2 if mode == ops.SWIGLU else self.out_features
        _, splits, scratch = ops.gemm_plan(tokens, features, self.in_features, mode)
        if splits <= 1:
            return None
        if scratch is not None:
            return ctx.buffer(scratch, (tokens, self.out_features), torch.float32)
        return ctx.buffer(out_name, (tokens, self.out_features), torch.float32)

    def _run(self, x, out, mode, ctx):
        if self._fast() and x.dtype == torch.bfloat16:
            scratch = ctx.buffer if ctx is not None else None
            cleared = ctx.take_cleared() if ctx is not None else False
            return ops.gemm(x, self.weight, out, mode, scratch=scratch, cleared=cleared)
        return ops.gemm_plain(x, self.weight, out, mode)
