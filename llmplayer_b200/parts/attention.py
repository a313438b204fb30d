"""Grouped-query softmax attention over the cached keys and values of each sequence.

One fused projection gives queries, keys and values; queries and keys are rotated
by the mixer's position encoding; keys and values are written to the sequence's
pages; every new token attends over the cache up to its own position (within the
window, if the layer has one); the output projection adds into the residual stream.

Reference: inference/Attention.java:76-240 (projections :86-114, rotation :129-131,
cache write :134-135, scale :138-140, scores/softmax/values :210-230, output
projection :234-239), GQA head mapping ``kvHead = h / (H/G)`` :212.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.sequence_cache import KVRequest
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, POSITIONS, Part, PendingNorm, Runtime
from .linear import Linear
from .specs import MATRIX, AttentionSpec, TensorSpec


class Attention(Part):
    def __init__(self, spec: AttentionSpec):
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ConfigError(f"{s.num_heads} query heads cannot share {s.num_kv_heads} key/value heads")
        if s.head_dim <= 0:
            raise ConfigError(f"head size {s.head_dim}")
        if s.window is not None and s.window <= 0:
            raise ConfigError(f"attention window must be positive or absent, got {s.window}")
        if not s.shares_kv and (s.k is None or s.v is None):
            raise ConfigError("an attention layer that keeps its own cache needs key and value projections")
        self.spec = spec
        self.position = POSITIONS.build(s.position)
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None

    @property
    def capture_safe(self) -> bool:
        # slots reach the kernels as page tables on the device; the position part must be safe as well
        return bool(getattr(self.position, "capture_safe", False))

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.spec
        specs = {s.q: TensorSpec((s.num_heads * s.head_dim, s.hidden_size), MATRIX)}
        if not s.shares_kv:
            specs[s.k] = TensorSpec((s.num_kv_heads * s.head_dim, s.hidden_size), MATRIX)
            specs[s.v] = TensorSpec((s.num_kv_heads * s.head_dim, s.hidden_size), MATRIX)
        specs[s.o] = TensorSpec((s.hidden_size, s.num_heads * s.head_dim), MATRIX)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().load(tensors, runtime)
        s = self.spec
        names = [s.q] if s.shares_kv else [s.q, s.k, s.v]
        self.qkv = Linear([tensors[n] for n in names], runtime)      # rows: queries, keys, values
        self.out = Linear([tensors[s.o]], runtime)
        self.position.load(tensors, runtime)

    # ------------------------------------------------------------------ cache
    def cache_request(self):
        s = self.spec
        if s.shares_kv:
            return None
        return KVRequest(s.num_kv_heads, s.head_dim, s.window)

    # ------------------------------------------------------------------ step
    def buffer_to_clear(self, ctx, tokens: int):
        return self.qkv.sums_into(ctx, tokens, "qkv", ops.STORE)

    takes_pending_norm = True     # the projection applies the norm of its input itself when a step is small

    def _forward_few(self, ctx, cache, pending: PendingNorm, residual: torch.Tensor, rotation) -> None:
        """A step of one token for each of a handful of sequences, in three kernels: projection of the
        normed stream (norm applied on the way in), rotation + cache write + attention, output projection.
        The projection's partial sums meet in a buffer that is zero between uses; it leaves each row's
        norm factor to the attention kernel and gives it the row's sum of squares instead."""
        s = self.spec
        T = residual.shape[0]
        H, G, hd = s.num_heads, s.num_kv_heads, s.head_dim
        F = self.qkv.out_features
        sums = ctx.workspace.get_zeroed("qkv_partial_sums", ops.FEW_TOKENS + ops.FEW_TOKENS * F)
        sumsq, qkv = sums[:ops.FEW_TOKENS], sums[ops.FEW_TOKENS:ops.FEW_TOKENS + T * F].view(T, F)
        with ops.section("attention.qkv"):
            deferred = self.qkv.few(pending.source, qkv, ops.STORE, norm=pending.norm, sumsq=sumsq)
        o = ctx.buffer("attn_out", (T, H * hd), torch.bfloat16)
        with ops.section("attention.scores"):
            ops.attention_decode_fused(
                qkv, rotation, o, cache.pages, ctx.page_tables[cache.group_index], ctx.kv_len, ctx.buffer,
                ctx.counters("decode_shares", ops.decode_groups(T, H, G)),
                num_heads=H, num_kv_heads=G, head_dim=hd, write_kv=not s.shares_kv, scale=s.scale, window=s.window,
                row_sumsq=sumsq if deferred else None, norm_eps=pending.norm.spec.eps, norm_width=residual.shape[1])
        with ops.section("attention.out"):
            self.out.few(o, residual, ops.ACCUMULATE, zero=sums[:ops.FEW_TOKENS + T * F])

    def forward(self, ctx, cache, x, residual: torch.Tensor, then_norm=None) -> bool:
        """Adds the layer's output into ``residual``; returns whether ``then_norm`` was fused.
        ``x``: the normed stream, or a :class:`PendingNorm` of it."""
        s, rt = self.spec, self.runtime
        if cache is None:
            raise ConfigError("attention needs a key/value cache (its own or another run's)")
        H, G, hd = s.num_heads, s.num_kv_heads, s.head_dim
        # the position encoding as something the kernels do on the way (a rotation), or None: then the
        # encoding's own part changes queries and keys in the projection's output before the kernels run
        rotation = self.position.rotation()
        if isinstance(x, PendingNorm):
            T = residual.shape[0]
            if (rt.fast and ctx.all_single and x.fusable and cache.pages.dtype == torch.bfloat16 and hd % 16 == 0
                    and hd <= 256 and self.qkv.can_few(T, ops.STORE) and self.out.can_few(T, ops.ACCUMULATE)
                    and residual.dtype == torch.float32 and rotation is not None):
                self._forward_few(ctx, cache, x, residual, rotation)
                return False
            x = x.tensor()
        T = x.shape[0]
        table = ctx.page_tables[cache.group_index]
        o = ctx.buffer("attn_out", (T, H * hd), rt.act_dtype)
        if (rt.fast and T >= ops.PERSISTENT_MIN_TOKENS and not ctx.all_single and rotation is not None
                and x.dtype == torch.bfloat16 and cache.pages.dtype == torch.bfloat16 and self.qkv.tensor_cores()
                and ops.qkv_rope_serves(rotation, hd)):
            # many tokens: the projection's epilogue rotates queries and keys and writes keys and values into the cache
            q = ctx.buffer("q", (T, H * hd), torch.bfloat16)
            with ops.section("attention.qkv"):
                ops.gemm_qkv_rope(x, self.qkv.weight, ctx.angles(rotation) if rotation.rotary_dim else None,
                                  rotation.interleaved, ctx.positions, ctx.seq_ids, table, q,
                                  None if s.shares_kv else cache.pages, num_heads=H, num_kv_heads=G, head_dim=hd)
            with ops.section("attention.scores"):
                ops.attention(ctx, q, o, cache.pages, table, num_heads=H, num_kv_heads=G, head_dim=hd,
                              scale=s.scale, window=s.window, fast=True)
            with ops.section("attention.out"):
                return self.out.accumulate(o, residual, ctx, then_norm)
        qkv = ctx.buffer("qkv", (T, self.qkv.out_features), torch.float32)
        with ops.section("attention.qkv"):
            self.qkv.store(x, qkv, ctx)
        if rotation is None:
            with ops.section("attention.position"):
                self.position.apply(ctx, qkv, num_heads=H, num_kv_heads=0 if s.shares_kv else G, head_dim=hd)
            rotation = ops.NO_ROTATION
        if rt.fast and ctx.all_single and cache.pages.dtype == torch.bfloat16 and hd % 16 == 0 and hd <= 256:
            # one token per sequence: rotation, cache write, attention and the merge of its shares in one kernel
            with ops.section("attention.scores"):
                ops.attention_decode_fused(
                    qkv, rotation, o, cache.pages, table, ctx.kv_len, ctx.buffer,
                    ctx.counters("decode_shares", ops.decode_groups(T, H, G)), num_heads=H,
                    num_kv_heads=G, head_dim=hd, write_kv=not s.shares_kv, scale=s.scale, window=s.window)
            with ops.section("attention.out"):
                return self.out.accumulate(o, residual, ctx, then_norm)
        q = ctx.buffer("q", (T, H * hd), rt.act_dtype)
        with ops.section("attention.position"):
            ops.rope_cache_write(
                qkv, rotation, ctx.positions, ctx.seq_ids, table, q,
                None if s.shares_kv else cache.pages,
                num_heads=H, num_kv_heads=G, head_dim=hd)
        with ops.section("attention.scores"):
            ops.attention(ctx, q, o, cache.pages, table, num_heads=H, num_kv_heads=G, head_dim=hd,
                          scale=s.scale, window=s.window, fast=rt.fast)
        with ops.section("attention.out"):
            return self.out.accumulate(o, residual, ctx, then_norm)


MIXERS.register("attention", Attention)
