"""The decode-attention entry point that allocates nothing, called through its exported C
symbol as a user without an allocator would call it, against the regular entry point.

Collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes
import math

import pytest
import torch

from test_kernel_attention import build_cache

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 4 << 20


def declare(lib):
    fn = lib.lp_attention_decode_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, P, I, P, I, I, I, I, I, ctypes.c_float, I, I, I, P]
    fn.restype = I
    return fn


def one_case(seed, lengths, H, G, hd, window, splits):
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    _, pages, table = build_cache(lengths, G, hd, torch.bfloat16, seed)
    g = torch.Generator().manual_seed(seed + 7)
    B = len(lengths)
    q = torch.randn(B, H * hd, generator=g).to(torch.bfloat16).to(dev)
    pages, table = pages.to(dev), table.to(dev)
    kv_len = torch.tensor(lengths, dtype=torch.int32, device=dev)
    per = -(-table.shape[1] // splits)
    n_splits = -(-table.shape[1] // per)
    kw = dict(num_heads=H, num_kv_heads=G, head_dim=hd, scale=1.0 / math.sqrt(hd), window=window)

    expected = torch.zeros_like(q)
    ops.attention_decode(q, expected, pages, table, kv_len,
                         lambda name, shape, dt: torch.empty(shape, dtype=dt, device=dev),
                         pages_per_split=per, num_splits=n_splits, **kw)

    lib = ops.library("attention_mma")
    fn = declare(lib)
    got = torch.full_like(q, 3.0)
    code = fn(q.data_ptr(), got.data_ptr(), pages.data_ptr(), table.data_ptr(), table.shape[1], kv_len.data_ptr(),
              B, H, G, hd, pages.shape[3], 1.0 / math.sqrt(hd), window or 0, per, n_splits,
              torch.cuda.current_stream().cuda_stream)
    assert code == 0, lib.lp_last_error().decode()
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    err = float((got.float() - expected.float()).abs().max())
    assert err <= 2e-2, err          # the tolerance of the attention tests; in practice the results are equal
    return err


def test_two_calls_in_a_row_match_the_regular_entry_point():
    # the second call is smaller and differently shaped: whatever the first left in the array must not show
    first = one_case(11, [700, 65, 1, 129, 300], H=8, G=2, hd=64, window=None, splits=4)
    second = one_case(12, [40, 333], H=6, G=3, hd=48, window=70, splits=2)
    assert first == 0.0 and second == 0.0


def test_requests_beyond_the_built_in_array_are_refused():
    from llmplayer_b200.kernels import ops
    lib = ops.library("attention_mma")
    fn = declare(lib)
    dev = "cuda:0"
    B, H, G, hd, splits = 64, 128, 8, 128, 8                     # 64*128*8*130 floats > 4 Mi
    assert B * H * splits * (hd + 2) > SCRATCH_FLOATS
    dummy = torch.zeros(16, dtype=torch.int32, device=dev)
    code = fn(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 1, dummy.data_ptr(),
              B, H, G, hd, 64, 0.1, 0, 1, splits, torch.cuda.current_stream().cuda_stream)
    assert code == -1
    message = lib.lp_last_error().decode()
    assert "floats of scratch" in message and str(SCRATCH_FLOATS) in message
    torch.cuda.synchronize()                                     # nothing was launched, the context is fine
