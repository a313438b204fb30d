"""The operations of a step, as calls into the compiled CUDA libraries.

Each function checks the tensors it is given (device, dtype, shape, layout),
then launches on torch's current stream. There is no other implementation
behind them: without a GPU and the compiled library they raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..errors import ExtensionMissing, KernelError
from . import build

F32, BF16 = 0, 1
STORE, ACCUMULATE, SWIGLU = 0, 1, 2
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_P, _I, _F = c_void_p, c_int, c_float
_SIGNATURES = {
    "elementwise": {
        "lp_embed": [_P, _I, _P, _P, _I, _I, _P],
        "lp_rmsnorm": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _F, _P, ctypes.c_longlong, _P],
        "lp_rope_cache_write": [_P, _I, _P, _P, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
        "lp_advance": [_P, _P, _P, _P, _I, _P],
        "lp_rope_angles": [_P, _P, _P, _I, _I, _P],
    },
    "gemm_plain": {
        "lp_gemm_plain": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    },
    "attention_plain": {
        "lp_attention_plain": [_P, _P, _I, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    },
    "gemm_tcgen05": {
        "lp_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P,
                            ctypes.c_longlong, _P, _P],
        "lp_gemm_persistent": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "lp_gemm_fewtok": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _F, _P, _P, _I, _P],
        "lp_gemm_configure": [_I, _I, _I, _I, _I],
        "lp_gemm_qkv_rope": [_P, _P, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    },
    "attention_mma": {
        "lp_attention_prefill": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P],
        "lp_attention_decode": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
        "lp_attention_decode_fitted": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
        "lp_attention_decode_fused": [_P, _I, _P, _I, _I, _P, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I,
                                      _I, _I, _I, _P, _F, _I, ctypes.c_longlong, _P, _P],
    },
    "attention_tcgen05": {
        "lp_attention_prefill_tc": [_P, _P, _P, ctypes.c_longlong, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I,
                                    _P, _P],
    },
    "host_loop": {
        "lp_decode_loop": [_P, _P, _P, _I, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P],
        "lp_decode_loop_sampled": [_P, _P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P,
                                   _P, _P, _P, _P, _P, _P],
    },
    "sampling": {
        "lp_sample": [_P, ctypes.c_longlong, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P],
        "lp_sample_params_size": [],
        "lp_sample_select_words": [],
        "lp_sample_slice_capacity": [_I],
        "lp_argmax": [_P, ctypes.c_longlong, _I, _I, _P, _P, _P],
        "lp_sample_fetch": [_P, _P, _I, _I, _I, _I, _P],
    },
}

_libs: Dict[str, ctypes.CDLL] = {}


def _env_int(name: str, default: int) -> int:
    import os
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


@dataclass
class KernelSettings:
    """Switches of the kernels, one set per process (the compiled libraries are shared by every engine of the
    process). The defaults are what was measured best; the environment variables of the same meaning
    (``LLMPLAYER_B200_PDL``, ``_FEW_TOKENS``, ``_FEWTOK``, ``_RING_SHARED``, ``_RING_ALONE``) set the initial
    values, :func:`configure` (which the engine's options call) changes them.

    ``pdl``: programmatic dependent launch between the kernels of a step. ``few_tokens``: up to how many tokens
    the parts put the RMS norm inside the consuming product and use the few-token kernel. ``fewtok_kernel``:
    whether 16-token tiles of the general product go to the mma.sync few-token kernel. ``ring_shared`` /
    ``ring_alone``: stages of that kernel's ring when two CTAs share an SM / when a CTA has one to itself.
    ``ring_alone_tile``: the most stages the one-tile tcgen05 product takes when its grid has no more CTAs than SMs
    (0, the default: never more than what lets two CTAs share an SM; a deeper ring measured slower).
    ``ring_normed``: the same for the tcgen05 product with the norm on the way in (9 to 64 tokens), whose stages
    also hold a float32 tile of x; there the deeper ring measured faster."""
    pdl: bool = True
    few_tokens: int = 32
    fewtok_kernel: bool = True
    ring_shared: int = 6
    ring_alone: int = 10
    ring_alone_tile: int = 0
    ring_normed: int = 6

    @classmethod
    def from_env(cls) -> "KernelSettings":
        return cls(pdl=_env_int("LLMPLAYER_B200_PDL", 1) != 0, few_tokens=_env_int("LLMPLAYER_B200_FEW_TOKENS", 32),
                   fewtok_kernel=_env_int("LLMPLAYER_B200_FEWTOK", 1) != 0,
                   ring_shared=_env_int("LLMPLAYER_B200_RING_SHARED", 6),
                   ring_alone=_env_int("LLMPLAYER_B200_RING_ALONE", 10),
                   ring_alone_tile=_env_int("LLMPLAYER_B200_RING_ALONE_TILE", 0),
                   ring_normed=_env_int("LLMPLAYER_B200_RING_NORMED", 6))


settings = KernelSettings.from_env()


def _apply_settings(name: str, lib: ctypes.CDLL) -> None:
    lib.lp_set_pdl.argtypes = [c_int]
    lib.lp_set_pdl.restype = None
    lib.lp_set_pdl(1 if settings.pdl else 0)
    if name == "gemm_tcgen05":
        lib.lp_gemm_configure(1 if settings.fewtok_kernel else 0, int(settings.ring_shared), int(settings.ring_alone),
                              int(settings.ring_alone_tile), int(settings.ring_normed))


def configure(**changes) -> KernelSettings:
    """Change kernel settings (fields of :class:`KernelSettings`) for this process, now and for libraries
    loaded later. Graphs captured before the change keep what they were captured with."""
    global FEW_TOKENS
    for key, value in changes.items():
        if value is None:
            continue
        if not hasattr(settings, key):
            raise KernelError(f"unknown kernel setting {key!r}")
        setattr(settings, key, type(getattr(settings, key))(value))
    FEW_TOKENS = max(0, min(int(settings.few_tokens), FEW_TOKENS_MAX))
    for name, lib in _libs.items():
        _apply_settings(name, lib)
    return settings


def library(name: str) -> ctypes.CDLL:
    """The loaded library ``name``; compiled first if it is missing or stale."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    path = build.ensure_built(name)
    try:
        lib = ctypes.CDLL(path)
    except OSError as exc:
        raise ExtensionMissing(f"cannot load {path}: {exc}") from None
    for fn, args in _SIGNATURES.get(name, {}).items():
        f = getattr(lib, fn)
        f.argtypes = args
        f.restype = c_int
    lib.lp_last_error.restype = ctypes.c_char_p
    _apply_settings(name, lib)
    _libs[name] = lib
    return lib


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise ExtensionMissing("no CUDA device: this library runs on the GPU only and has no CPU path")


# --------------------------------------------------------------------------- profile mode
class _NoSection:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SECTION = _NoSection()


class StepProfiler:
    """Device time per section of the model walk, from CUDA-event pairs around each section.

    The reference's ``-Dcuda.profile=true`` puts stream barriers between the sections of a token's forward
    pass and prints milliseconds per section (java21 inference/CudaForwardPass.java:1431-1456, :1646-1737);
    graph replay is off meanwhile (:1761). Here a section is a ``with ops.section(name):`` block in a part;
    the events between sections also keep neighbouring kernels from overlapping, so the times add up to
    the step's, and steps run directly instead of from captured graphs."""

    def __init__(self):
        self._pairs = []            # (name, start event, end event), resolved when a report is asked for
        self._totals: Dict[str, list] = {}
        self.steps = 0

    class _Section:
        def __init__(self, owner, name):
            self.owner, self.name = owner, name

        def __enter__(self):
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
            return self

        def __exit__(self, *exc):
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.owner._pairs.append((self.name, self.start, end))
            return False

    def section(self, name: str):
        return StepProfiler._Section(self, name)

    def _resolve(self) -> None:
        if self._pairs:
            torch.cuda.synchronize()
            for name, start, end in self._pairs:
                entry = self._totals.setdefault(name, [0.0, 0])
                entry[0] += start.elapsed_time(end)
                entry[1] += 1
            self._pairs = []

    def report(self) -> dict:
        """{"steps": n, "total_ms": t, "sections": {name: {"ms": total, "calls": c, "ms_per_step": m}}}"""
        self._resolve()
        steps = max(1, self.steps)
        sections = {name: {"ms": ms, "calls": calls, "ms_per_step": ms / steps}
                    for name, (ms, calls) in sorted(self._totals.items(), key=lambda kv: -kv[1][0])}
        return {"steps": self.steps, "total_ms": sum(v["ms"] for v in sections.values()), "sections": sections}

    def reset(self) -> None:
        self._resolve()
        self._totals = {}
        self.steps = 0


_profiler: Optional[StepProfiler] = None


def set_profiler(profiler: Optional[StepProfiler]) -> None:
    global _profiler
    _profiler = profiler


def section(name: str):
    """``with ops.section("attention.qkv"):`` around the launches of one section of the model walk; costs
    nothing unless a profiler is set."""
    return _NO_SECTION if _profiler is None else _profiler.section(name)


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched by this process."""
    return _launches


def count_launches(n: int) -> None:
    """Kernels launched by replaying captured graphs from native code (the host loop) are counted here."""
    global _launches
    _launches += int(n)


def _check(lib: ctypes.CDLL, code: int) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(lib.lp_last_error().decode("utf-8", "replace") or f"kernel call failed with code {code}")


_device_index = None


def current_stream() -> int:
    return _stream()


def _stream() -> int:
    """The raw handle of torch's current stream (asked of torch's C layer directly: this is on the path of
    every launch)."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    try:
        return torch._C._cuda_getCurrentRawStream(_device_index)
    except AttributeError:                        # a torch without that entry
        return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _want(t: torch.Tensor, what: str, dtype=None, ndim: Optional[int] = None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: expected a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected dtype {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{what}: expected {ndim} dimensions, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: expected a contiguous tensor, got strides {t.stride()}")
    return t


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------- embedding
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = float32(table[tokens[t], :])."""
    _want(table, "embed table", ndim=2)
    _want(tokens, "embed tokens", torch.int32, 1)
    _want(out, "embed out", torch.float32, 2)
    T, d = out.shape
    if tokens.numel() != T or table.shape[1] != d:
        raise KernelError(f"embed: {tokens.numel()} tokens, table {tuple(table.shape)}, out {tuple(out.shape)}")
    lib = library("elementwise")
    _check(lib, lib.lp_embed(table.data_ptr(), _code(table, "embed table"), tokens.data_ptr(), out.data_ptr(),
                             T, d, _stream()))
    return out


# --------------------------------------------------------------------------- norm
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None,
            clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = x[rows[r]] / sqrt(mean(x^2) + eps) * weight, float32 inside.

    ``add`` (same shape as x) is first added into x in place: the residual sum
    fused with the norm that follows it. ``clear``: a float32 buffer that is set to
    zero on the side (for a product after the norm that sums partial results into it).
    """
    _want(x, "rmsnorm x", torch.float32, 2)
    _want(weight, "rmsnorm weight", torch.float32, 1)
    _want(out, "rmsnorm out", ndim=2)
    d = x.shape[1]
    R = out.shape[0]
    if weight.numel() != d or out.shape[1] != d:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _want(rows, "rmsnorm rows", torch.int32, 1)
        if rows.numel() != R:
            raise KernelError(f"rmsnorm: {rows.numel()} row indices for {R} output rows")
    elif x.shape[0] != R:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)} and out {tuple(out.shape)} differ in rows")
    add_code = F32
    if add is not None:
        _want(add, "rmsnorm add", ndim=2)
        if add.shape != x.shape:
            raise KernelError(f"rmsnorm: add {tuple(add.shape)} does not match x {tuple(x.shape)}")
        add_code = _code(add, "rmsnorm add")
    if clear is not None:
        _want(clear, "rmsnorm clear", torch.float32)
    lib = library("elementwise")
    _check(lib, lib.lp_rmsnorm(x.data_ptr(), _ptr(add), add_code, _ptr(rows), weight.data_ptr(), out.data_ptr(),
                               _code(out, "rmsnorm out"), R, d, float(eps), _ptr(clear),
                               clear.numel() if clear is not None else 0, _stream()))
    return out


# --------------------------------------------------------------------------- rotation + cache write
@dataclass(frozen=True)
class Rotation:
    """What the kernels that prepare queries and keys can do to them on the way: rotate the first
    ``rotary_dim`` features of every head by ``position * inv_freq[pair]``, the pairs being
    (i, i + rotary_dim / 2) or, ``interleaved``, (2i, 2i + 1). ``rotary_dim == 0``: nothing.
    A position encoding that is such a rotation hands this to the kernels; any other rule is
    applied by its own part before they run."""
    inv_freq: Optional[torch.Tensor] = None      # float32 [rotary_dim / 2] on the device
    rotary_dim: int = 0
    interleaved: bool = False

    def checked(self, what: str):
        """(pointer or None, rotary_dim, interleaved as int) after checking the frequencies."""
        if self.rotary_dim <= 0:
            return None, 0, 0
        _want(self.inv_freq, f"{what} inv_freq", torch.float32, 1)
        if self.inv_freq.numel() != self.rotary_dim // 2:
            raise KernelError(f"{what}: {self.inv_freq.numel()} frequencies for a rotary width of {self.rotary_dim}")
        return self.inv_freq.data_ptr(), int(self.rotary_dim), 1 if self.interleaved else 0


NO_ROTATION = Rotation()


def rope_cache_write(qkv: torch.Tensor, rotation: Rotation, positions: torch.Tensor,
                     seq_ids: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor,
                     pages: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Rotate queries (and keys), write queries to ``q_out`` [T, H*hd] and keys and
    values into ``pages`` [num_pages, 2, G, page_size, hd]. ``pages=None``: queries only."""
    _want(qkv, "rope qkv", torch.float32, 2)
    _want(positions, "rope positions", torch.int32, 1)
    _want(seq_ids, "rope seq_ids", torch.int32, 1)
    _want(page_table, "rope page_table", torch.int32, 2)
    _want(q_out, "rope q_out", ndim=2)
    T = qkv.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if positions.numel() != T or seq_ids.numel() != T or q_out.shape != (T, H * hd):
        raise KernelError(f"rope: qkv {tuple(qkv.shape)}, q_out {tuple(q_out.shape)}, {positions.numel()} positions")
    page_size, kv_code = 0, F32
    if pages is not None:
        _want(pages, "rope pages", ndim=5)
        if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
            raise KernelError(f"rope: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
        page_size, kv_code = pages.shape[3], _code(pages, "rope pages")
    freq_ptr, rotary_dim, interleaved = rotation.checked("rope")
    lib = library("elementwise")
    _check(lib, lib.lp_rope_cache_write(
        qkv.data_ptr(), qkv.shape[1], freq_ptr, positions.data_ptr(),
        seq_ids.data_ptr(), page_table.data_ptr(), page_table.shape[1], q_out.data_ptr(), _code(q_out, "rope q_out"),
        _ptr(pages), kv_code, T, H, G, hd, rotary_dim, interleaved, page_size, _stream()))


def rope_angles(positions: torch.Tensor, rotation: Rotation, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = (cos, sin) of float(positions[t]) * inv_freq[i], float32 [T, rotary_dim / 2, 2]: the angles of a
    step's tokens, formed once for a product whose epilogue rotates (:func:`gemm_qkv_rope`)."""
    _want(positions, "rope_angles positions", torch.int32, 1)
    _want(out, "rope_angles out", torch.float32, 3)
    freq_ptr, rotary_dim, _ = rotation.checked("rope_angles")
    T, half = positions.numel(), rotary_dim // 2
    if out.shape != (T, half, 2) or half == 0:
        raise KernelError(f"rope_angles: out {tuple(out.shape)} for {T} tokens and a rotary width of {rotary_dim}")
    lib = library("elementwise")
    _check(lib, lib.lp_rope_angles(positions.data_ptr(), freq_ptr, out.data_ptr(), T, half, _stream()))
    return out


QKV_ROPE_HEAD_SIZES = (32, 64, 128, 256)


def qkv_rope_serves(rotation: Rotation, head_dim: int) -> bool:
    """Whether :func:`gemm_qkv_rope` can apply this rotation to heads of this size in its epilogue."""
    if head_dim not in QKV_ROPE_HEAD_SIZES or rotation.rotary_dim not in (0, head_dim):
        return False
    return rotation.rotary_dim == 0 or rotation.interleaved or head_dim >= 64


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, angles: Optional[torch.Tensor], interleaved: bool,
                  positions: torch.Tensor, seq_ids: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor,
                  pages: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """The fused projection of a step with many tokens on the tensor cores, with what follows it in its epilogue:
    ``x`` [T, K] x ``w`` [(H + 2G) * hd, K]^T (rows of queries, keys, values; ``[H * hd, K]`` and ``pages=None``
    for a layer without keys of its own), queries and keys rotated by ``angles`` (from :func:`rope_angles`;
    None: no rotation), queries written to ``q_out`` [T, H * hd], keys and values into ``pages`` at the tokens'
    positions. All bfloat16."""
    _want(x, "gemm_qkv_rope x", torch.bfloat16, 2)
    _want(w, "gemm_qkv_rope w", torch.bfloat16, 2)
    _want(q_out, "gemm_qkv_rope q_out", torch.bfloat16, 2)
    _want(positions, "gemm_qkv_rope positions", torch.int32, 1)
    _want(seq_ids, "gemm_qkv_rope seq_ids", torch.int32, 1)
    _want(page_table, "gemm_qkv_rope page_table", torch.int32, 2)
    T, K = x.shape
    H, G, hd = num_heads, num_kv_heads, head_dim
    heads = H + 2 * G if pages is not None else H
    if w.shape != (heads * hd, K) or q_out.shape != (T, H * hd) or positions.numel() != T or seq_ids.numel() != T:
        raise KernelError(f"gemm_qkv_rope: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)}")
    page_size = 0
    if pages is not None:
        _want(pages, "gemm_qkv_rope pages", torch.bfloat16, 5)
        if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
            raise KernelError(f"gemm_qkv_rope: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
        page_size = pages.shape[3]
    half = 0
    if angles is not None:
        _want(angles, "gemm_qkv_rope angles", torch.float32, 3)
        half = angles.shape[1]
        if angles.shape != (T, half, 2):
            raise KernelError(f"gemm_qkv_rope: angles {tuple(angles.shape)} for {T} tokens")
    lib = library("gemm_tcgen05")
    _check(lib, lib.lp_gemm_qkv_rope(
        x.data_ptr(), w.data_ptr(), T, K, K, K, _ptr(angles), half, 1 if interleaved else 0, positions.data_ptr(),
        seq_ids.data_ptr(), page_table.data_ptr(), page_table.shape[1], q_out.data_ptr(), _ptr(pages), H, G, hd,
        page_size, kernel_status().data_ptr(), _stream()))


# --------------------------------------------------------------------------- matrix products
def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STORE) -> torch.Tensor:
    """out (=|+=) a @ w.T with float32 multiply-adds in increasing k.

    ``SWIGLU``: ``w`` is [2N, K], gate rows then up rows; out = silu(a gate^T) * (a up^T).
    """
    _want(a, "gemm a", ndim=2)
    _want(w, "gemm w", ndim=2)
    _want(out, "gemm out", ndim=2)
    M, K = a.shape
    N = out.shape[1]
    rows = 2 * N if mode == SWIGLU else N
    if w.shape != (rows, K) or out.shape[0] != M:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, mode {mode}")
    lib = library("gemm_plain")
    _check(lib, lib.lp_gemm_plain(a.data_ptr(), _code(a, "gemm a"), w.data_ptr(), _code(w, "gemm w"), out.data_ptr(),
                                  _code(out, "gemm out"), M, N, K, K, K, N, mode, _stream()))
    return out


_num_sms = None


def num_sms() -> int:
    """Streaming multiprocessors of the current device (asked once)."""
    global _num_sms
    if _num_sms is None:
        require_gpu()
        _num_sms = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return _num_sms


_status = None


def kernel_status() -> torch.Tensor:
    """One int32 in device memory that kernels with bounded waits set when a wait runs out."""
    global _status
    if _status is None:
        _status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _status


def check_kernel_status() -> None:
    """Raise if a kernel reported a wait that ran out. Reads the word back, which synchronises."""
    if _status is not None and int(_status.item()) != 0:
        code = int(_status.item())
        _status.zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting on a barrier (code {code}: "
                          "1 = loader, 2 = MMA issuer, 3 = epilogue, 4-5 = operand maker; 2x the same in the "
                          "persistent product; 6 = a page of the decode attention)")


def _token_tile(tokens: int, gated: bool) -> int:
    # up to 64 tokens: the smallest tile that holds them; beyond: 128, of which two CTAs share an SM
    # (so one's epilogue runs under the other's MMAs); 256 remains available to callers
    for tile in (16, 32, 64):
        if tokens <= tile:
            return tile
    return 128


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """The weight layout of the tensor-core gated product: for every 64 output features, their 64
    gate rows followed by their 64 up rows (features padded with zero rows to a multiple of 64)."""
    F, K = gate.shape
    if up.shape != gate.shape:
        raise KernelError(f"gate {tuple(gate.shape)} and up {tuple(up.shape)} differ")
    pad = -F % 64
    if pad:
        zeros = torch.zeros((pad, K), dtype=gate.dtype, device=gate.device)
        gate, up = torch.cat([gate, zeros]), torch.cat([up, zeros])
    blocks = (F + pad) // 64
    return torch.stack([gate.view(blocks, 64, K), up.view(blocks, 64, K)], dim=1).reshape(2 * (F + pad), K).contiguous()


def gemm_plan(tokens: int, features: int, k: int, mode: int):
    """(token tile, splits) that :func:`gemm` uses for these sizes."""
    k_blocks = -(-k // 64)
    tile = _token_tile(tokens, mode == SWIGLU)
    if mode == SWIGLU:
        return tile, 1
    ctas = -(-features // 128) * -(-tokens // tile)
    sms = num_sms()
    if ctas >= sms // 2 or k_blocks < 8:
        return tile, 1
    return tile, max(1, min(sms // ctas, k_blocks // 4))


FUSED_NORM_MAX_TOKENS = 4
PERSISTENT_MIN_TOKENS = 512


def _persistent_pays(tokens: int, features: int, k: int, mode: int) -> bool:
    """Whether the persistent form (one CTA per SM walking 128 x 256 tiles, 128 x 128 x 2 when gated)
    fills the SMs at least as well as separate CTAs of 128 x 128 tiles, two to an SM."""
    feat_tiles = -(-features // 128)
    persistent_tiles = feat_tiles * -(-tokens // (128 if mode == SWIGLU else 256))
    separate_ctas = feat_tiles * -(-tokens // 128)
    sms = num_sms()
    fill_p = persistent_tiles / (-(-persistent_tiles // sms) * sms)
    fill_s = separate_ctas / (-(-separate_ctas // (2 * sms)) * 2 * sms)
    # at equal fill the persistent form wins when the SMs are well filled (its tiles are twice as large and one
    # tile's epilogue hides under the next one's MMAs) or the K loop is long
    return fill_p > fill_s + 0.02 or (fill_p >= fill_s and (fill_p >= 0.8 or k >= 4096))


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STORE, *, block_tok: int = 0,
         splits: int = 0, cleared: bool = False, norm_after=None) -> torch.Tensor:
    """out (=|+=) a @ w.T on the tensor cores (bfloat16 in, float32 accumulation).

    ``a`` [tokens, K] and ``w`` [features, K] are bfloat16; for ``SWIGLU``, ``w`` is the
    interleaved gate/up matrix of :func:`interleave_gate_up` and ``out`` [tokens, features] gets
    silu(gate) * up. When few CTAs would cover the output, the K range is split over more of
    them and the partial sums meet in float32 atomics; ``cleared`` says that ``out`` is already
    zero for that. ``block_tok`` / ``splits`` override the plan (tests).

    ``norm_after = (gain, eps, normed_out, clear, counter)`` (``ACCUMULATE`` only, at most
    ``FUSED_NORM_MAX_TOKENS`` rows): once all CTAs have added their parts, the last one writes
    the RMS norm of every row of ``out`` to ``normed_out`` (bfloat16) and zeroes ``clear``
    (a float32 tensor or None). ``counter``: one int32 on the device that is zero between uses
    (the CTAs count themselves there; the last one sets it back).
    """
    _want(a, "gemm a", torch.bfloat16, 2)
    _want(w, "gemm w", torch.bfloat16, 2)
    _want(out, "gemm out", ndim=2)
    M, K = a.shape
    N = out.shape[1]
    rows = 128 * (-(-N // 64)) if mode == SWIGLU else N
    if w.shape != (rows, K) or out.shape[0] != M:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, mode {mode}")
    if M == 0:
        return out
    lib = library("gemm_tcgen05")
    status = kernel_status()
    if (M >= PERSISTENT_MIN_TOKENS and not block_tok and not splits and norm_after is None
            and _persistent_pays(M, N, K, mode)):
        # many tokens: one CTA per SM walks over the tiles, epilogue and MMAs of neighbouring tiles overlap
        if mode == ACCUMULATE and out.dtype != torch.float32:
            raise KernelError("gemm: accumulation needs a float32 output")
        _check(lib, lib.lp_gemm_persistent(a.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out, "gemm out"), M, N, K,
                                           K, K, N, mode, status.data_ptr(), _stream()))
        return out
    tile, n_splits = gemm_plan(M, N, K, mode)
    tile = block_tok or tile
    n_splits = 1 if mode == SWIGLU else (splits or n_splits)
    if mode == ACCUMULATE:
        if out.dtype != torch.float32:
            raise KernelError("gemm: accumulation needs a float32 output")
    elif mode == STORE and n_splits > 1:
        if out.dtype != torch.float32:
            n_splits = 1
        elif not cleared:
            out.zero_()
    norm_args = (None, 0.0, None, None, 0, None)
    if norm_after is not None:
        gain, eps, normed, clear, counter = norm_after
        if mode != ACCUMULATE or M > FUSED_NORM_MAX_TOKENS:
            raise KernelError("gemm: a following norm needs an accumulating product of few rows")
        _want(gain, "gemm norm gain", torch.float32, 1)
        _want(normed, "gemm normed out", torch.bfloat16, 2)
        if gain.numel() != N or normed.shape != (M, N):
            raise KernelError(f"gemm: norm gain {tuple(gain.shape)}, normed out {tuple(normed.shape)} for [{M}, {N}]")
        if clear is not None:
            _want(clear, "gemm norm clear", torch.float32)
        _want(counter, "gemm norm counter", torch.int32, 1)
        norm_args = (gain.data_ptr(), float(eps), normed.data_ptr(), _ptr(clear),
                     clear.numel() if clear is not None else 0, counter.data_ptr())
    _check(lib, lib.lp_gemm_tcgen05(a.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out, "gemm out"), M, N, K,
                                    K, K, N, mode, tile, n_splits, status.data_ptr(), *norm_args, _stream()))
    return out


FEW_TOKENS_MAX = 64                  # what the few-token entry takes
# Up to where the parts choose it with the norm inside (``settings.few_tokens``). Measured at the 1B shape (ms per
# step, norm inside against separate norm kernels): 8 tokens 0.68 / 0.76 (the mma.sync kernel); 12 tokens
# 0.79 / 0.87, 16 tokens 0.80 / 0.88, 20 tokens 0.84 / 0.89, 32 tokens 0.86 / 0.94 (the tcgen05 kernel with operand
# makers); 48 tokens 1.07 / 0.99 and 64 tokens 1.14 / 1.06: beyond 32 tokens the norm kernels stay.
FEW_TOKENS = max(0, min(int(settings.few_tokens), FEW_TOKENS_MAX))


def gemm_few(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STORE, *, norm=None,
             sumsq: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None) -> bool:
    """out (=|+=) f(x) @ w.T for at most ``FEW_TOKENS_MAX`` rows, with what a decode step fuses around it
    (up to 16 rows, 8 with a norm, the mma.sync kernel; beyond that the one-tile tcgen05 kernels).

    ``norm = (gain, eps)``: ``x`` is the float32 residual stream and the product applies the RMS norm on
    the way in. If the K range is then shared out over CTAs (few output features), ``out`` still lacks each
    row's factor: ``sumsq`` [rows] (zero beforehand) receives the rows' sums of squares, the reader applies
    ``1 / sqrt(sumsq / K + eps)``, and the function returns True. ``out`` must be zero beforehand in that
    case, as for any ``STORE`` whose partial sums meet in atomics. ``zero``: a float32 buffer cleared on the
    side. Without ``norm``, ``x`` is bfloat16."""
    _want(w, "gemm_few w", torch.bfloat16, 2)
    _want(out, "gemm_few out", ndim=2)
    _want(x, "gemm_few x", torch.float32 if norm is not None else torch.bfloat16, 2)
    M, K = x.shape
    N = out.shape[1]
    rows = 128 * (-(-N // 64)) if mode == SWIGLU else N
    if w.shape != (rows, K) or out.shape[0] != M or M > FEW_TOKENS_MAX:
        raise KernelError(f"gemm_few: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, mode {mode}")
    _, splits = gemm_plan(M, N, K, mode)
    if mode == STORE and splits > 1 and out.dtype != torch.float32:
        splits = 1
    gain = eps = None
    if norm is not None:
        gain, eps = norm
        _want(gain, "gemm_few gain", torch.float32, 1)
        if gain.numel() != K:
            raise KernelError(f"gemm_few: a gain of {gain.numel()} values for rows of {K}")
        if splits > 1 and sumsq is None:
            splits = 1
    deferred = norm is not None and splits > 1
    if deferred:
        _want(sumsq, "gemm_few sumsq", torch.float32, 1)
        if sumsq.numel() < M:
            raise KernelError(f"gemm_few: {sumsq.numel()} sums of squares for {M} rows")
    if zero is not None:
        _want(zero, "gemm_few zero", torch.float32)
    lib = library("gemm_tcgen05")
    _check(lib, lib.lp_gemm_fewtok(
        x.data_ptr(), _code(x, "gemm_few x"), w.data_ptr(), out.data_ptr(), _code(out, "gemm_few out"), M, N, K, K, K, N,
        mode, splits, kernel_status().data_ptr(), _ptr(gain), float(eps) if eps is not None else 0.0,
        sumsq.data_ptr() if deferred else None, _ptr(zero), zero.numel() if zero is not None else 0, _stream()))
    return deferred


# --------------------------------------------------------------------------- attention
def attention_plain(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor,
                    seq_ids: torch.Tensor, positions: torch.Tensor, *, num_heads: int, num_kv_heads: int,
                    head_dim: int, scale: float, window: Optional[int]) -> torch.Tensor:
    """Each query token attends over the cached keys of its sequence up to its own
    position (and within ``window``, if given)."""
    _want(q, "attention q", ndim=2)
    _want(out, "attention out", q.dtype, 2)
    _want(pages, "attention pages", ndim=5)
    _want(page_table, "attention page_table", torch.int32, 2)
    _want(seq_ids, "attention seq_ids", torch.int32, 1)
    _want(positions, "attention positions", torch.int32, 1)
    T = q.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if q.shape != (T, H * hd) or out.shape != q.shape or seq_ids.numel() != T or positions.numel() != T:
        raise KernelError(f"attention: q {tuple(q.shape)}, out {tuple(out.shape)} for {H} heads of {hd}")
    if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
        raise KernelError(f"attention: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
    lib = library("attention_plain")
    _check(lib, lib.lp_attention_plain(
        q.data_ptr(), out.data_ptr(), _code(q, "attention q"), pages.data_ptr(), _code(pages, "attention pages"),
        page_table.data_ptr(), page_table.shape[1], seq_ids.data_ptr(), positions.data_ptr(), T, H, G, hd,
        pages.shape[3], float(scale), int(window) if window else 0, _stream()))
    return out


def _check_attention(q, out, pages, page_table, H, G, hd, what):
    _want(q, f"{what} q", torch.bfloat16, 2)
    _want(out, f"{what} out", torch.bfloat16, 2)
    _want(pages, f"{what} pages", torch.bfloat16, 5)
    _want(page_table, f"{what} page_table", torch.int32, 2)
    if q.shape[1] != H * hd or out.shape != q.shape:
        raise KernelError(f"{what}: q {tuple(q.shape)}, out {tuple(out.shape)} for {H} heads of {hd}")
    if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
        raise KernelError(f"{what}: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")


tcgen05_attention = True      # tests switch it off to reach the mma.sync kernel at every size


def attention_prefill(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor,
                      q_start: torch.Tensor, kv_len: torch.Tensor, max_new: int, *, num_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: Optional[int]) -> torch.Tensor:
    """Tensor-core attention for a step that brings several tokens per sequence.
    ``q_start`` [B+1]: offsets of each sequence's new tokens; ``kv_len`` [B]: lengths after the step."""
    _check_attention(q, out, pages, page_table, num_heads, num_kv_heads, head_dim, "attention_prefill")
    _want(q_start, "attention_prefill q_start", torch.int32, 1)
    _want(kv_len, "attention_prefill kv_len", torch.int32, 1)
    B = kv_len.numel()
    if q_start.numel() != B + 1 or page_table.shape[0] != B:
        raise KernelError(f"attention_prefill: {B} sequences, {q_start.numel()} offsets, table {tuple(page_table.shape)}")
    if head_dim in (64, 128) and max_new > 64 and tcgen05_attention:
        # long runs of new tokens with heads of 64 or 128: scores and P V on the tcgen05 tensor cores
        lib = library("attention_tcgen05")
        _check(lib, lib.lp_attention_prefill_tc(
            q.data_ptr(), out.data_ptr(), pages.data_ptr(), pages.shape[0], page_table.data_ptr(),
            page_table.shape[1], q_start.data_ptr(), kv_len.data_ptr(), B, q.shape[0], int(max_new), num_heads,
            num_kv_heads, head_dim, pages.shape[3], float(scale), int(window) if window else 0,
            kernel_status().data_ptr(), _stream()))
        return out
    lib = library("attention_mma")
    _check(lib, lib.lp_attention_prefill(
        q.data_ptr(), out.data_ptr(), pages.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        q_start.data_ptr(), kv_len.data_ptr(), B, int(max_new), num_heads, num_kv_heads, head_dim, pages.shape[3],
        float(scale), int(window) if window else 0, _stream()))
    return out


MIN_SHARE_PAGES = 8
LONG_SHARE_PAGES = 14


def decode_split(batch: int, num_kv_heads: int, num_heads: int, table_width: int):
    """How a decode step's pages are shared out over CTAs: (pages per share, shares) for page tables of
    ``table_width`` entries. A share and the merge of shares cost several dependent round trips to memory, so a
    sequence is cut only into shares of at least ``MIN_SHARE_PAGES`` pages, and into no more CTAs than there are SMs
    (the kernel then gives each CTA 16 warps), or twice that for shares of twice the pages. This is the most shares
    a sequence can get; the kernels fit the
    number to each sequence's own length (at batch 8 and a context of 600 in a table of 16 pages: one share,
    0.69 ms per step, against 0.75 with two shares of 8 pages)."""
    groups = decode_groups(batch, num_heads, num_kv_heads)
    shares = max(1, min(table_width // MIN_SHARE_PAGES, num_sms() // groups))
    # long sequences: up to two CTAs per SM (8 warps each) if every share still has LONG_SHARE_PAGES pages. Measured with the pages
    # brought by TMA, ms per step at contexts of 3.5 k / 1 k: batch 4: 0.771 -> 0.756 / 0.716 -> 0.711, batch 8:
    # 0.837 -> 0.818 / unchanged, batch 16: 1.080 -> 1.048 / 0.828 (0.856 with shares of 8 pages there)
    shares = max(shares, min(table_width // LONG_SHARE_PAGES, 2 * num_sms() // groups))
    per = -(-table_width // shares)
    return per, -(-table_width // per)


def attention_decode(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor,
                     kv_len: torch.Tensor, scratch, *, num_heads: int, num_kv_heads: int, head_dim: int,
                     scale: float, window: Optional[int], pages_per_split: int = 0, num_splits: int = 0) -> torch.Tensor:
    """Tensor-core attention for a step of one token per sequence. ``scratch(name, shape, dtype)``
    supplies the float32 buffer for the partial results of the shares."""
    _check_attention(q, out, pages, page_table, num_heads, num_kv_heads, head_dim, "attention_decode")
    _want(kv_len, "attention_decode kv_len", torch.int32, 1)
    B = kv_len.numel()
    if q.shape[0] != B or page_table.shape[0] != B:
        raise KernelError(f"attention_decode: {B} sequences, q {tuple(q.shape)}, table {tuple(page_table.shape)}")
    fitted = not pages_per_split or not num_splits
    if fitted:
        pages_per_split, num_splits = decode_split(B, num_kv_heads, num_heads, page_table.shape[1])
    buf = scratch("attention_partials", (B * num_heads * num_splits * (head_dim + 2),), torch.float32)
    lib = library("attention_mma")
    if fitted:
        _check(lib, lib.lp_attention_decode_fitted(
            q.data_ptr(), out.data_ptr(), pages.data_ptr(), page_table.data_ptr(), page_table.shape[1],
            kv_len.data_ptr(), buf.data_ptr(), B, num_heads, num_kv_heads, head_dim, pages.shape[3], float(scale),
            int(window) if window else 0, num_splits, MIN_SHARE_PAGES, _stream()))
        return out
    _check(lib, lib.lp_attention_decode(
        q.data_ptr(), out.data_ptr(), pages.data_ptr(), page_table.data_ptr(), page_table.shape[1], kv_len.data_ptr(),
        buf.data_ptr(), B, num_heads, num_kv_heads, head_dim, pages.shape[3], float(scale),
        int(window) if window else 0, pages_per_split, num_splits, _stream()))
    return out


DECODE_HEAD_ROWS = 8          # query heads that one CTA of a decode step serves (HEAD_ROWS of the kernels)


def decode_groups(batch: int, num_heads: int, num_kv_heads: int) -> int:
    """How many groups of CTAs a fused decode step has (each merges its own shares and counts them in a
    counter of its own)."""
    return batch * num_kv_heads * (-(-(num_heads // num_kv_heads) // DECODE_HEAD_ROWS))


def attention_decode_fused(qkv: torch.Tensor, rotation: Rotation, out: torch.Tensor,
                           pages: torch.Tensor, page_table: torch.Tensor, kv_len: torch.Tensor, scratch,
                           counters: torch.Tensor, *,
                           num_heads: int, num_kv_heads: int, head_dim: int,
                           write_kv: bool, scale: float, window: Optional[int], pages_per_split: int = 0,
                           num_splits: int = 0, row_sumsq: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                           norm_width: int = 0) -> torch.Tensor:
    """A decode step's attention from the float32 fused projection ``qkv`` [B, (H + 2G) * hd]
    (``[B, H * hd]`` when ``write_kv`` is false): rotates the queries, rotates and stores the new
    key, stores the new value, attends over the pages and merges the shares, in one kernel.
    ``counters``: int32, at least ``decode_groups(B, H, G)`` entries, zero between uses (the shares of a
    group count themselves there and the last one sets the counter back).
    Without ``pages_per_split`` / ``num_splits`` the shares are fitted to each sequence's own length.
    ``row_sumsq`` [B]: ``qkv`` still lacks the factor of the RMS norm of its input; row b is scaled by
    ``1 / sqrt(row_sumsq[b] / norm_width + norm_eps)`` as it is read."""
    _want(qkv, "attention_decode_fused qkv", torch.float32, 2)
    _want(out, "attention_decode_fused out", torch.bfloat16, 2)
    _want(pages, "attention_decode_fused pages", torch.bfloat16, 5)
    _want(page_table, "attention_decode_fused page_table", torch.int32, 2)
    _want(kv_len, "attention_decode_fused kv_len", torch.int32, 1)
    _want(counters, "attention_decode_fused counters", torch.int32, 1)
    H, G, hd = num_heads, num_kv_heads, head_dim
    B = kv_len.numel()
    heads = H + 2 * G if write_kv else H
    if qkv.shape != (B, heads * hd) or out.shape != (B, H * hd) or page_table.shape[0] != B:
        raise KernelError(f"attention_decode_fused: qkv {tuple(qkv.shape)}, out {tuple(out.shape)}, {B} sequences")
    if pages.shape[1] != 2 or pages.shape[2] != G or pages.shape[4] != hd:
        raise KernelError(f"attention_decode_fused: pages {tuple(pages.shape)} do not fit {G} key heads of {hd}")
    freq_ptr, rotary_dim, interleaved = rotation.checked("attention_decode_fused")
    fitted = not pages_per_split or not num_splits
    if fitted:                       # as many shares as the tables allow; the kernel fits them to each sequence
        _, num_splits = decode_split(B, G, H, page_table.shape[1])
        pages_per_split = page_table.shape[1]
    if counters.numel() < decode_groups(B, H, G):
        raise KernelError(f"attention_decode_fused: {counters.numel()} counters for {decode_groups(B, H, G)} groups")
    buf = scratch("attention_partials", (B * H * num_splits * (hd + 2),), torch.float32)
    lib = library("attention_mma")
    _check(lib, lib.lp_attention_decode_fused(
        qkv.data_ptr(), qkv.shape[1], freq_ptr, rotary_dim, interleaved,
        out.data_ptr(), pages.data_ptr(), 1 if write_kv else 0, page_table.data_ptr(), page_table.shape[1],
        kv_len.data_ptr(), buf.data_ptr(), counters.data_ptr(), B, H, G, hd, pages.shape[3], float(scale),
        int(window) if window else 0, pages_per_split, num_splits, MIN_SHARE_PAGES if fitted else 0, _ptr(row_sumsq),
        float(norm_eps), int(norm_width), pages.shape[0], kernel_status().data_ptr(), _stream()))
    return out


def attention(ctx, q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, page_table: torch.Tensor, *,
              num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
              fast: bool) -> torch.Tensor:
    """Attention of the step's tokens over the cache; picks the kernel for the step's shape."""
    tensor_cores = (fast and q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16
                    and head_dim % 16 == 0 and head_dim <= 256)
    if tensor_cores and ctx.all_single:
        return attention_decode(q, out, pages, page_table, ctx.kv_len, ctx.buffer, num_heads=num_heads,
                                num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window)
    if tensor_cores:
        return attention_prefill(q, out, pages, page_table, ctx.q_start, ctx.kv_len, ctx.max_new,
                                 num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale,
                                 window=window)
    return attention_plain(q, out, pages, page_table, ctx.seq_ids, ctx.positions, num_heads=num_heads,
                           num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window)


# --------------------------------------------------------------------------- sampling
def sample_select_words() -> int:
    """4-byte words of scratch per row that ``sample`` wants for finding top-k candidates with several blocks."""
    return library("sampling").lp_sample_select_words()


def sample_slice_capacity(vocab: int) -> int:
    """The largest top-k whose candidates several blocks per row find together (0: none at this vocabulary)."""
    return library("sampling").lp_sample_slice_capacity(int(vocab))


def sample(logits: torch.Tensor, work: torch.Tensor, params: torch.Tensor, edit_token: torch.Tensor,
           edit_subtract: torch.Tensor, edit_factor: torch.Tensor, out_token: torch.Tensor,
           out_prob: torch.Tensor, select: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``params`` (packed LpSampleParams records) from the float32 ``logits``.
    ``select``: int32 scratch of ``sample_select_words()`` per row; with it, rows whose top-k is at most
    ``sample_slice_capacity(vocab)`` have their candidates found by several blocks each."""
    _want(logits, "sample logits", torch.float32, 2)
    _want(work, "sample work", torch.float32, 2)
    _want(params, "sample params", torch.uint8, 1)
    _want(edit_token, "sample edit tokens", torch.int32, 1)
    _want(edit_subtract, "sample edit amounts", torch.float32, 1)
    _want(edit_factor, "sample edit factors", torch.float32, 1)
    _want(out_token, "sample out tokens", torch.int32, 1)
    _want(out_prob, "sample out probabilities", torch.float32, 1)
    lib = library("sampling")
    record = lib.lp_sample_params_size()
    B = out_token.numel()
    V = logits.shape[1]
    if params.numel() != B * record or work.shape != (B, V) or out_prob.numel() != B:
        raise KernelError(f"sample: {params.numel()} parameter bytes, work {tuple(work.shape)} for {B} rows of {V}")
    select_ptr = 0
    if select is not None:
        _want(select, "sample select scratch", torch.int32, 1)
        if select.numel() < B * lib.lp_sample_select_words():
            raise KernelError(f"sample: select scratch of {select.numel()} words for {B} rows")
        select_ptr = select.data_ptr()
    _check(lib, lib.lp_sample(logits.data_ptr(), V, work.data_ptr(), V, params.data_ptr(), B, edit_token.data_ptr(),
                              edit_subtract.data_ptr(), edit_factor.data_ptr(), select_ptr, out_token.data_ptr(),
                              out_prob.data_ptr(), _stream()))


def sample_fetch(host_block: torch.Tensor, dev_block: torch.Tensor, batch: int, cap: int, record_words: int,
                 field_count: int) -> None:
    """Bring a step's sampler block (records, then ``cap`` edit tokens, amounts and factors per sequence) from
    page-locked host memory: each record and as many edits as it names."""
    _want(dev_block, "sample_fetch device block", torch.int32, 1)
    if host_block.dtype != torch.int32 or not host_block.is_pinned() or host_block.numel() != dev_block.numel():
        raise KernelError("sample_fetch: the host block must be page-locked int32 of the device block's size")
    if dev_block.numel() != batch * (record_words + 3 * cap):
        raise KernelError(f"sample_fetch: a block of {dev_block.numel()} words for {batch} records of {record_words} "
                          f"words and {cap} edits each")
    lib = library("sampling")
    _check(lib, lib.lp_sample_fetch(host_block.data_ptr(), dev_block.data_ptr(), batch, cap, record_words, field_count,
                                    _stream()))


def advance(tokens: torch.Tensor, positions: torch.Tensor, kv_len: torch.Tensor, sampled: torch.Tensor) -> None:
    """tokens <- sampled; positions += 1; kv_len += 1 (a decoding batch moves on by one token)."""
    B = tokens.numel()
    for t, what in ((tokens, "tokens"), (positions, "positions"), (kv_len, "kv_len"), (sampled, "sampled")):
        _want(t, f"advance {what}", torch.int32, 1)
        if t.numel() != B:
            raise KernelError(f"advance: {what} has {t.numel()} entries, tokens {B}")
    lib = library("elementwise")
    _check(lib, lib.lp_advance(tokens.data_ptr(), positions.data_ptr(), kv_len.data_ptr(), sampled.data_ptr(), B,
                               _stream()))


def argmax(logits: torch.Tensor, scratch: torch.Tensor, out_token: torch.Tensor) -> None:
    """out_token[b] = index of the first maximum of row b of the float32 ``logits``.
    ``scratch``: at least 64 float32 per row."""
    _want(logits, "argmax logits", torch.float32, 2)
    _want(scratch, "argmax scratch", torch.float32, 1)
    _want(out_token, "argmax out", torch.int32, 1)
    B, V = logits.shape
    if out_token.numel() != B or scratch.numel() < 64 * B:
        raise KernelError(f"argmax: {B} rows, {out_token.numel()} outputs, scratch of {scratch.numel()}")
    lib = library("sampling")
    _check(lib, lib.lp_argmax(logits.data_ptr(), V, V, B, scratch.data_ptr(), out_token.data_ptr(), _stream()))
