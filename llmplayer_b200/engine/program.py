"""A decode step as a list of operations for the persistent step kernel.

A step that brings one token for each of a few sequences is a chain of small
dependent operations. Run as separate kernels, each pays its launch and its first
round trip to memory; the persistent kernel (csrc/decode_program.cu) walks the same
chain inside one launch, with the weights of the next operation already on their way
while the CTAs meet at a barrier.

The parts write the list themselves: a part that can take part has an ``emit``
method beside ``forward`` and appends its operations to a :class:`StepProgram`
(products with an optional RMS norm of their input and a store / add / gated
epilogue; attention over the cache). A model whose parts all emit is run through the
program; any other model, and any step the program refuses (more tokens than the
kernel's tile, head sizes it has no unit for), runs through ``forward`` as before.

The reference replays a captured chain of one kernel per operation
(java21 inference/CudaForwardPass.java:1760-1812) and has no counterpart of this.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch

from ..kernels import ops

X_BF16, X_RMSNORM = 0, 1
STORE, ADD, SWIGLU = 0, 1, 2
MAX_OPERAND_BYTES = 128 * 1024


class ProgramRefused(Exception):
    """The step cannot be expressed as a program; the caller runs the chain of kernels instead."""


def max_tokens() -> int:
    return int(ops.library("decode_program").lp_program_max_tokens())


class StepProgram:
    def __init__(self, device: torch.device, tokens: int):
        self.lib = ops.library("decode_program")
        self.device = device
        self.tokens = int(tokens)
        if not 1 <= self.tokens <= self.lib.lp_program_max_tokens():
            raise ProgramRefused(f"{tokens} tokens in a step")
        self.grid = ops.NUM_SMS
        self._op_bytes = self.lib.lp_program_op_bytes()
        self._ops: List[ctypes.Array] = []
        self._clear_taken: List[bool] = []
        self._is_product: List[bool] = []
        self._last_use = {}                    # data_ptr -> index of the last operation that touches it
        self._keep: List[torch.Tensor] = []    # everything an operation points at stays alive with the program
        self._specs: List[dict] = []           # what each operation was built from ({} for attention)
        self.region_bytes = 0
        self._prologue: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None
        self._zero_at_start: Optional[torch.Tensor] = None
        self._device_ops: Optional[torch.Tensor] = None
        self._counter = torch.zeros(1, dtype=torch.int32, device=device)
        self._attn_counters: Optional[torch.Tensor] = None
        self.timing: Optional[torch.Tensor] = None      # int64 [ops, 4]: set to have CTA 0 stamp its clock per operation

    # ------------------------------------------------------------------ building
    def embed(self, table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor) -> None:
        """x[t] = float32(table[tokens[t]]): the step's first kernel."""
        if self._ops or self._prologue is not None:
            raise ProgramRefused("the embedding must come first")
        if table.dtype not in (torch.bfloat16, torch.float32) or x.dtype != torch.float32:
            raise ProgramRefused("embedding dtypes")
        self._prologue = (table, tokens, x)
        self._keep += [table, tokens, x]

    def _touch(self, *tensors: Optional[torch.Tensor]) -> None:
        for t in tensors:
            if t is not None:
                self._last_use[t.data_ptr()] = len(self._ops)

    def _choose_splits(self, feat_tiles: int, k_blocks: int) -> int:
        """Shares of K so that the units fill the grid: the fewest shares within a tenth of the best fill."""
        fills = {}
        for s in range(1, max(1, k_blocks // 2) + 1):
            units = feat_tiles * s
            fills[s] = units / (-(-units // self.grid) * self.grid)
        best = max(fills.values())
        return min(s for s, f in fills.items() if f >= 0.9 * best)

    def _zeroed_before(self, out: torch.Tensor) -> bool:
        """Arrange that ``out`` is zero when the operation about to be added starts: cleared by the
        CTAs during an earlier product that follows the buffer's last use by at least one barrier,
        or by the step's first kernel if nothing has used it yet."""
        here = len(self._ops)
        last = self._last_use.get(out.data_ptr())
        if last is None:
            if self._zero_at_start is None:
                self._zero_at_start = out
                return True
            return self._zero_at_start.data_ptr() == out.data_ptr() and self._zero_at_start.numel() >= out.numel()
        for j in range(last + 1, here):
            if self._is_product[j] and not self._clear_taken[j]:
                self._set_clear(j, out)
                return True
        return False

    def _set_clear(self, index: int, buf: torch.Tensor) -> None:
        # the fields `clear` and `clear_count` are rewritten through the library: rebuild is simplest
        spec = self._specs[index]
        spec["clear"] = buf
        self._ops[index] = self._encode_product(spec)
        self._clear_taken[index] = True

    def product(self, weight: torch.Tensor, *, x: torch.Tensor, out: torch.Tensor, epilogue: int,
                features: Optional[int] = None, norm=None, x_rows: Optional[torch.Tensor] = None,
                tokens: Optional[int] = None) -> None:
        """out (=|+=) f(x) @ weight.T for the step's tokens.

        ``norm = (gain, eps)``: x is float32 and each row is RMS-normed (and rounded to bfloat16)
        on its way into the product; otherwise x is bfloat16. ``epilogue``: STORE (float32),
        ADD (into float32) or SWIGLU (weight = interleaved gate/up rows, out bfloat16).
        ``x_rows``: int32 row numbers of x to use instead of 0..tokens-1."""
        n = self.tokens if tokens is None else int(tokens)
        if weight.dtype != torch.bfloat16 or weight.dim() != 2 or not weight.is_contiguous():
            raise ProgramRefused("weights must be contiguous bfloat16 matrices")
        rows, K = weight.shape
        if K % 8:
            raise ProgramRefused(f"K = {K}")
        if norm is not None:
            if x.dtype != torch.float32:
                raise ProgramRefused("a normed operand starts from float32")
        elif x.dtype != torch.bfloat16:
            raise ProgramRefused("an operand without norm must be bfloat16")
        if x.shape[-1] != K or x.stride(-1) != 1:
            raise ProgramRefused("operand width")
        want_out = torch.bfloat16 if epilogue == SWIGLU else torch.float32
        if out.dtype != want_out or out.stride(-1) != 1:
            raise ProgramRefused("output dtype")
        feats = int(features) if features is not None else rows
        k_blocks = -(-K // 64)
        feat_tiles = -(-rows // 128)
        splits = 1
        if epilogue == ADD or (epilogue == STORE and feat_tiles < self.grid // 2):
            splits = self._choose_splits(feat_tiles, k_blocks)
        if epilogue == STORE and splits > 1:
            # partial sums meet in atomics: the output must be zero first
            if self._zeroed_before(out):
                epilogue = ADD
            else:
                splits = 1
        while -(-k_blocks // splits) * self.lib.lp_program_operand_bytes(1) > MAX_OPERAND_BYTES:
            if epilogue != ADD or splits >= k_blocks:
                raise ProgramRefused(f"an operand of {K} columns does not fit shared memory")
            splits += 1
        self.region_bytes = max(self.region_bytes, self.lib.lp_program_operand_bytes(-(-k_blocks // splits)))
        spec = dict(weight=weight, features=feats, splits=splits, x=x, x_rows=x_rows, norm=norm, tokens=n,
                    epilogue=epilogue, out=out, clear=None)
        self._touch(x, out)
        self._specs.append(spec)
        self._ops.append(self._encode_product(spec))
        self._clear_taken.append(False)
        self._is_product.append(True)
        self._keep += [t for t in (weight, x, out, x_rows) + (tuple(norm[:1]) if norm else ()) if t is not None]

    def _encode_product(self, spec: dict) -> ctypes.Array:
        w, x, out = spec["weight"], spec["x"], spec["out"]
        norm = spec["norm"]
        clear = spec["clear"]
        buf = (ctypes.c_uint8 * self._op_bytes)()
        code = self.lib.lp_program_product(
            ctypes.addressof(buf), w.data_ptr(), w.shape[0], w.shape[1], w.stride(0), spec["features"], spec["splits"],
            X_RMSNORM if norm is not None else X_BF16, x.data_ptr(), x.stride(-2) if x.dim() > 1 else x.shape[-1],
            ops._ptr(spec["x_rows"]), norm[0].data_ptr() if norm is not None else None,
            float(norm[1]) if norm is not None else 0.0, spec["tokens"], spec["epilogue"], out.data_ptr(),
            out.stride(-2) if out.dim() > 1 else out.shape[-1], ops._ptr(clear),
            clear.numel() if clear is not None else 0)
        if code != 0:
            raise ProgramRefused(self.lib.lp_last_error().decode("utf-8", "replace"))
        return buf

    def attention(self, *, qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
                  out: torch.Tensor, pages: torch.Tensor, write_kv: bool, page_table: torch.Tensor,
                  kv_len: torch.Tensor, scratch, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                  window: Optional[int]) -> None:
        """Rotation, cache write and attention of the step's tokens, from the float32 fused projection."""
        H, G, hd = num_heads, num_kv_heads, head_dim
        B = kv_len.numel()
        if B != self.tokens or pages.dtype != torch.bfloat16 or qkv.dtype != torch.float32 or out.dtype != torch.bfloat16:
            raise ProgramRefused("attention operands")
        if hd not in (64, 128):
            raise ProgramRefused(f"heads of {hd}")
        width = page_table.shape[1]
        groups = B * G * (-(-(H // G) // 16))
        # a share and the merge of shares cost a few dependent round trips to L2: worth it from 8 pages each
        shares = max(1, min(width // 8, self.grid // max(groups, 1)))
        per = -(-width // shares)
        shares = -(-width // per)
        partials = scratch("program_attention_partials", (B * H * shares * (hd + 2),), torch.float32)
        if self._attn_counters is None or self._attn_counters.numel() < groups:
            self._attn_counters = torch.zeros(max(groups, 1024), dtype=torch.int32, device=self.device)
        buf = (ctypes.c_uint8 * self._op_bytes)()
        code = self.lib.lp_program_attention(
            ctypes.addressof(buf), qkv.data_ptr(), qkv.shape[1], ops._ptr(inv_freq) if rotary_dim > 0 else None,
            int(rotary_dim), 1 if interleaved else 0, out.data_ptr(), pages.data_ptr(), 1 if write_kv else 0,
            page_table.data_ptr(), width, kv_len.data_ptr(), partials.data_ptr(), self._attn_counters.data_ptr(),
            B, H, G, hd, pages.shape[3], float(scale), int(window) if window else 0, per, shares)
        if code != 0:
            raise ProgramRefused(self.lib.lp_last_error().decode("utf-8", "replace"))
        self.region_bytes = max(self.region_bytes, self.lib.lp_program_attention_bytes(hd))
        self._touch(qkv, out)
        self._specs.append({})
        self._ops.append(buf)
        self._clear_taken.append(True)
        self._is_product.append(False)
        self._keep += [qkv, out, pages, page_table, kv_len, partials] + ([inv_freq] if inv_freq is not None else [])

    # ------------------------------------------------------------------ running
    def finish(self) -> "StepProgram":
        if self._prologue is None or not self._ops:
            raise ProgramRefused("an empty program")
        blob = b"".join(bytes(b) for b in self._ops)
        host = torch.frombuffer(bytearray(blob), dtype=torch.uint8)
        self._device_ops = host.to(self.device)
        if self._device_ops.data_ptr() % 128:
            raise ProgramRefused("operation list alignment")
        return self

    def run(self) -> None:
        """The step: the embedding kernel, then the persistent kernel, on the current stream."""
        table, tokens, x = self._prologue
        zero = self._zero_at_start
        stream = ops._stream()
        ops._check(self.lib, self.lib.lp_program_prologue(
            table.data_ptr(), ops._code(table, "embedding table"), tokens.data_ptr(), x.data_ptr(), x.shape[0],
            x.shape[1], table.shape[0], ops._ptr(zero), zero.numel() if zero is not None else 0,
            self._counter.data_ptr(), stream))
        ops._check(self.lib, self.lib.lp_program_launch(
            self._device_ops.data_ptr(), len(self._ops), self.grid, self.region_bytes, self._counter.data_ptr(),
            ops.kernel_status().data_ptr(), ops._ptr(self.timing), stream))

    def describe(self) -> str:
        lines = []
        for i, spec in enumerate(self._specs):
            if spec:
                w = spec["weight"]
                lines.append(f"{i:3d} product {tuple(w.shape)} shares {spec['splits']} epilogue {spec['epilogue']}"
                             f"{' norm' if spec['norm'] else ''}{' +clear' if spec['clear'] is not None else ''}")
            else:
                lines.append(f"{i:3d} attention")
        return "\n".join(lines)
