"""The attention kernels alone (plain, tensor-core prefill, tensor-core decode) against a
float64 softmax attention, on caches whose pages are scattered and partly stale."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

PAGE = 64
# Largest |kernel - float64 attention| allowed in bfloat16, on outputs of order one: at most four times the worst
# that each kernel achieved on a B200 (decode and fused decode 4.3e-3, prompt kernels 1.0e-2, plain kernel 7.8e-3).
BOUND = {"decode": 1.5e-2, "fused": 1.5e-2, "prefill": 2e-2, "plain": 2e-2}


def build_cache(lengths, G, hd, dtype, seed, extra_pages=5):
    """Dense K/V per sequence plus their scattered paged form. Unused rows hold large junk."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // PAGE) for n in lengths]
    num_pages = sum(need) + extra_pages
    order = torch.randperm(num_pages, generator=g).tolist()
    pages = (torch.randn(num_pages, 2, G, PAGE, hd, generator=g) * 30.0).to(dtype)      # junk everywhere
    width = max(need)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    dense = []
    for b, n in enumerate(lengths):
        k = torch.randn(n, G, hd, generator=g).to(dtype)
        v = torch.randn(n, G, hd, generator=g).to(dtype)
        dense.append((k, v))
        for blk in range(need[b]):
            page = order.pop()
            table[b, blk] = page
            rows = slice(blk * PAGE, min(n, (blk + 1) * PAGE))
            cnt = rows.stop - rows.start
            pages[page, 0, :, :cnt] = k[rows].transpose(0, 1)
            pages[page, 1, :, :cnt] = v[rows].transpose(0, 1)
    return dense, pages, table


def reference(q, k, v, positions, scale, window):
    """q [Tq, H, hd]; k, v [Tk, G, hd] (positions 0..Tk-1); float64 softmax attention."""
    q, k, v = q.double(), k.double(), v.double()
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros_like(q)
    t = torch.arange(k.shape[0])
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        ok = t[None, :] <= positions[:, None]
        if window:
            ok &= t[None, :] > positions[:, None] - window
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def run_case(kind, lengths, new, H, G, hd, window, dtype, seed=0, crafted=False, shares=None):
    """``new[b]`` tokens of sequence b are the step's queries (the last ``new[b]`` positions).
    ``shares``: into how many shares a decode kernel cuts the page tables (None: its own choice);
    ``kind="fused"`` runs the decode kernel that starts from the projection (no rotation, no cache write)."""
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    dense, pages, table = build_cache(lengths, G, hd, dtype, seed)
    g = torch.Generator().manual_seed(seed + 1)
    T = sum(new)
    q = torch.randn(T, H, hd, generator=g).to(dtype)
    positions, seq_ids, q_start = [], [], [0]
    for b, (n, m) in enumerate(zip(lengths, new)):
        positions += list(range(n - m, n))
        seq_ids += [b] * m
        q_start.append(q_start[-1] + m)
    positions = torch.tensor(positions)
    if crafted:
        # one far key must win: scale a query and a key at the far end of each sequence's context
        for b, (n, m) in enumerate(zip(lengths, new)):
            far = 1 if not window else max(0, n - window)      # just inside the window's edge
            k, v = dense[b]
            row = q_start[b] + m - 1
            q[row] = 0
            q[row, :, 0] = 16.0
            k[far] = 0
            k[far, :, 0] = 16.0
            blk, off = divmod(far, PAGE)
            pages[table[b, blk], 0, :, off] = k[far]
    ref = torch.cat([reference(q[q_start[b]:q_start[b + 1]], dense[b][0], dense[b][1],
                               positions[q_start[b]:q_start[b + 1]], 1.0 / math.sqrt(hd), window)
                     for b in range(len(lengths))])
    qd = q.reshape(T, H * hd).to(dev)
    out = torch.full_like(qd, 7.0)
    pages_d, table_d = pages.to(dev), table.to(dev)
    kw = dict(num_heads=H, num_kv_heads=G, head_dim=hd, scale=1.0 / math.sqrt(hd), window=window)
    kv_len = torch.tensor(lengths, dtype=torch.int32, device=dev)
    if kind == "plain":
        ops.attention_plain(qd, out, pages_d, table_d, torch.tensor(seq_ids, dtype=torch.int32, device=dev),
                            positions.to(torch.int32).to(dev), **kw)
    elif kind == "prefill":
        ops.attention_prefill(qd, out, pages_d, table_d, torch.tensor(q_start, dtype=torch.int32, device=dev), kv_len,
                              max(new), **kw)
    else:
        assert all(m == 1 for m in new)
        scratch = {}

        def buf(name, shape, dt):
            scratch[name] = torch.full(shape, float("nan"), dtype=dt, device=dev)
            return scratch[name]
        split = {}
        if shares:
            per = -(-table.shape[1] // shares)
            split = dict(pages_per_split=per, num_splits=-(-table.shape[1] // per))
        if kind == "fused":
            # the queries as the float32 projection would deliver them; this layer keeps no keys of its own, so
            # the kernel attends over the pages as they are
            counters = torch.zeros(ops.decode_groups(len(lengths), H, G), dtype=torch.int32, device=dev)
            ops.attention_decode_fused(qd.float(), ops.NO_ROTATION, out, pages_d, table_d, kv_len, buf, counters,
                                       write_kv=False, **kw, **split)
            assert int(counters.abs().sum()) == 0
        else:
            ops.attention_decode(qd, out, pages_d, table_d, kv_len, buf, **kw, **split)
    torch.cuda.synchronize()
    got = out.reshape(T, H, hd).double().cpu()
    assert torch.isfinite(got).all()
    err = float((got - ref).abs().max())
    from helpers import record_error
    record_error(f"attention kernel ({kind}), {str(dtype).split('.')[-1]}", f"H{H} G{G} hd{hd} window {window}", err,
                 2e-5 if dtype == torch.float32 else BOUND.get(kind, 2e-2))
    if crafted:
        for b in range(len(lengths)):
            row = q_start[b + 1] - 1
            far = 1 if not window else max(0, lengths[b] - window)
            want = dense[b][1][far].double()            # the far key dominates: output = its value
            H_G = H // G
            for h in range(H):
                assert (got[row, h] - want[h // H_G]).abs().max() < 0.05, (b, h)
    return err


GEOMETRIES = [(4, 2, 16), (3, 1, 32), (6, 3, 48), (32, 8, 64), (8, 2, 128), (2, 2, 256), (20, 1, 64)]


@pytest.mark.parametrize("H,G,hd", GEOMETRIES)
@pytest.mark.parametrize("window", [None, 70])
def test_plain_attention(H, G, hd, window):
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        err = run_case("plain", [1, 64, 65, 300], [1, 64, 3, 150], H, G, hd, window, dtype)
        assert err < tol, err


@pytest.mark.parametrize("H,G,hd", GEOMETRIES)
@pytest.mark.parametrize("window", [None, 70])
def test_tensor_core_prefill(H, G, hd, window):
    """Heads of 64 with long runs of new tokens take the tcgen05 kernel, everything else mma.sync."""
    err = run_case("prefill", [1, 64, 65, 300, 129], [1, 64, 3, 150, 129], H, G, hd, window, torch.bfloat16)
    assert err < BOUND["prefill"], err


@pytest.mark.parametrize("H,G,hd", [(32, 8, 64), (20, 1, 64), (3, 3, 64), (8, 2, 128), (24, 8, 128), (5, 5, 128)])
@pytest.mark.parametrize("window", [None, 70, 200])
@pytest.mark.parametrize("tcgen05", [True, False])
def test_both_prefill_kernels_at_head_sizes_64_and_128(H, G, hd, window, tcgen05, monkeypatch):
    from llmplayer_b200.kernels import ops
    monkeypatch.setattr(ops, "tcgen05_attention", tcgen05)
    lengths, new = [700, 128, 129, 391, 65], [700, 128, 100, 130, 65]        # whole prompts and continued ones
    err = run_case("prefill", lengths, new, H, G, hd, window, torch.bfloat16, seed=7)
    assert err < BOUND["prefill"], err
    run_case("prefill", [900, 333], [200, 70], H, G, hd, window, torch.bfloat16, seed=3, crafted=True)


@pytest.mark.parametrize("hd", [64, 128])
def test_prefill_whose_maximum_keeps_growing(hd):
    """The tcgen05 prompt kernel keeps a reference maximum per row that moves only when the row's true maximum
    has outgrown it by a factor of 256; here every later page holds a key that beats all earlier ones by far more
    (and by less, in alternation), so the output in tensor memory is brought down again and again."""
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    H, G, n = 4, 2, 640
    dense, pages, table = build_cache([n], G, hd, torch.bfloat16, seed=5)
    k, v = dense[0]
    g = torch.Generator().manual_seed(6)
    q = torch.randn(n, H, hd, generator=g).to(torch.bfloat16)
    q[:, :, 0] = 4.0
    for page in range(n // PAGE):                      # one key per page whose score grows page by page
        at = page * PAGE + 17
        k[at] = 0
        k[at, :, 0] = (1.5 if page % 2 else 6.0) * (page + 1)
        pages[table[0, page], 0, :, 17] = k[at]
    ref = reference(q, k, v, torch.arange(n), 1.0 / math.sqrt(hd), None)
    qd = q.reshape(n, H * hd).to(dev)
    out = torch.zeros_like(qd)
    ops.attention_prefill(qd, out, pages.to(dev), table.to(dev), torch.tensor([0, n], dtype=torch.int32, device=dev),
                          torch.tensor([n], dtype=torch.int32, device=dev), n, num_heads=H, num_kv_heads=G, head_dim=hd,
                          scale=1.0 / math.sqrt(hd), window=None)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    err = float((out.reshape(n, H, hd).double().cpu() - ref).abs().max())
    assert err < BOUND["prefill"], err


@pytest.mark.parametrize("H,G,hd", GEOMETRIES)
@pytest.mark.parametrize("window", [None, 70])
def test_tensor_core_decode(H, G, hd, window):
    lengths = [1, 64, 65, 700, 129, 17]
    err = run_case("decode", lengths, [1] * len(lengths), H, G, hd, window, torch.bfloat16)
    assert err < BOUND["decode"], err


@pytest.mark.parametrize("kind", ["decode", "fused"])
@pytest.mark.parametrize("shares", [2, 3, 5])
@pytest.mark.parametrize("window", [None, 70, 200])
def test_decode_in_several_shares_against_float64(kind, shares, window):
    """The pages of a sequence cut into shares: with a window some shares lie wholly before it, one share may
    hold nothing but the newest page, short sequences leave most shares empty. Compared with the float64
    attention (not with another entry point of the same kernel), random and with one far key made to win."""
    lengths = [1, 64, 65, 700, 129, 17, 641]
    err = run_case(kind, lengths, [1] * len(lengths), 8, 2, 64, window, torch.bfloat16, seed=11, shares=shares)
    assert err < BOUND[kind], err
    err = run_case(kind, lengths, [1] * len(lengths), 6, 3, 48, window, torch.bfloat16, seed=12, shares=shares)
    assert err < BOUND[kind], err
    run_case(kind, [900, 333, 70], [1, 1, 1], 8, 2, 64, window, torch.bfloat16, seed=3, crafted=True, shares=shares)


@pytest.mark.parametrize("kind", ["decode", "fused"])
@pytest.mark.parametrize("window", [None, 300, 1000])
def test_shares_fitted_to_each_sequence(kind, window):
    """Left to themselves the decode kernels cut every sequence into as many shares as its own length (within the
    window) gives pages for: here four, two, one and one shares in one grid, some CTAs with nothing to do."""
    lengths = [2000, 70, 1100, 513]
    err = run_case(kind, lengths, [1] * 4, 8, 2, 64, window, torch.bfloat16, seed=31)
    assert err < BOUND[kind], err
    run_case(kind, lengths, [1] * 4, 4, 2, 128, window, torch.bfloat16, seed=32, crafted=True)


def test_a_sequence_of_length_zero_reads_and_writes_nothing():
    """A row whose length is zero is an empty sequence: its output is zero, and neither its neighbours'
    results nor any page changes (the fused kernel stores no key for it)."""
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    H, G, hd = 8, 2, 64
    lengths = [130, 0, 65]
    _, pages, table = build_cache([130, 1, 65], G, hd, torch.bfloat16, seed=21)
    g = torch.Generator().manual_seed(22)
    qkv = torch.randn(3, (H + 2 * G) * hd, generator=g).to(dev)
    table_d = table.to(dev)
    kw = dict(num_heads=H, num_kv_heads=G, head_dim=hd, scale=hd ** -0.5, window=None)

    def scratch(name, shape, dt):
        return torch.full(shape, float("nan"), dtype=dt, device=dev)

    def run(lens, shares):
        p = pages.to(dev).clone()
        out = torch.full((3, H * hd), 5.0, dtype=torch.bfloat16, device=dev)
        counters = torch.zeros(ops.decode_groups(3, H, G), dtype=torch.int32, device=dev)
        per = -(-table.shape[1] // shares)
        ops.attention_decode_fused(qkv, ops.NO_ROTATION, out, p, table_d,
                                   torch.tensor(lens, dtype=torch.int32, device=dev), scratch, counters,
                                   write_kv=True, pages_per_split=per, num_splits=-(-table.shape[1] // per), **kw)
        torch.cuda.synchronize()
        return out, p

    for shares in (1, 3):
        with_empty, pages_empty = run(lengths, shares)
        with_one, pages_one = run([130, 1, 65], shares)
        assert torch.isfinite(with_empty.float()).all()
        assert float(with_empty[1].float().abs().max()) == 0.0
        assert torch.equal(with_empty[0], with_one[0]) and torch.equal(with_empty[2], with_one[2])
        # only the page of the middle sequence may differ between the two runs, and with a length of zero
        # it is exactly what it was
        middle = int(table[1, 0])
        assert torch.equal(pages_empty[middle], pages.to(dev)[middle])
        others = [i for i in range(pages.shape[0]) if i != middle]
        assert torch.equal(pages_empty[others], pages_one[others])
    q = torch.randn(3, H * hd, generator=g).to(torch.bfloat16).to(dev)
    out = torch.full_like(q, 5.0)
    ops.attention_decode(q, out, pages.to(dev), table_d, torch.tensor(lengths, dtype=torch.int32, device=dev), scratch,
                         pages_per_split=1, num_splits=table.shape[1], **kw)
    torch.cuda.synchronize()
    assert float(out[1].float().abs().max()) == 0.0 and torch.isfinite(out.float()).all()


def test_shared_memory_grants_do_not_cross_between_head_sizes():
    """Each kernel instantiation remembers its own grant of dynamic shared memory: a decode step at a head
    size of 96 (which needs a large grant) must not make the kernel for heads of 64 skip asking for its own."""
    for hd in (96, 64, 112, 128, 64):
        for kind in ("decode", "fused"):
            err = run_case(kind, [700, 65], [1, 1], 4, 2, hd, None, torch.bfloat16, seed=hd, shares=2)
            assert err < BOUND[kind], (hd, kind, err)


@pytest.mark.parametrize("kind", ["plain", "prefill", "decode"])
@pytest.mark.parametrize("window", [None, 200])
def test_a_far_key_among_hundreds_is_found(kind, window):
    lengths = [900, 333]
    new = [1, 1] if kind == "decode" else [5, 1]
    run_case(kind, lengths, new, 8, 2, 64, window, torch.bfloat16, seed=3, crafted=True)


@pytest.mark.parametrize("H,G,hd,rd,pairing", [(32, 8, 64, 64, "split_half"), (6, 3, 48, 32, "interleaved"),
                                               (20, 1, 64, 64, "split_half"), (4, 2, 128, 0, "split_half")])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("splits", [1, 3])
def test_fused_decode_equals_rotation_then_attention(H, G, hd, rd, pairing, window, splits):
    """The fused decode kernel (rotation, cache write, attention, merge) against the separate kernels."""
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    lengths = [1, 64, 65, 700, 129, 17]
    B = len(lengths)
    _, pages, table = build_cache(lengths, G, hd, torch.bfloat16, seed=hd + H)
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, (H + 2 * G) * hd, generator=g).to(dev)
    inv = (torch.rand(max(rd // 2, 1), generator=g) * 0.5).to(dev) if rd else None
    table_d = table.to(dev)
    kv_len = torch.tensor(lengths, dtype=torch.int32, device=dev)
    positions = kv_len - 1
    seq_ids = torch.arange(B, dtype=torch.int32, device=dev)
    kw = dict(num_heads=H, num_kv_heads=G, head_dim=hd)
    per = -(-table.shape[1] // splits)
    n_splits = -(-table.shape[1] // per)

    def scratch(name, shape, dt):
        return torch.full(shape, float("nan"), dtype=dt, device=dev)

    pages_a = pages.to(dev).clone()
    q = torch.empty(B, H * hd, dtype=torch.bfloat16, device=dev)
    rotation = ops.Rotation(inv, rd, pairing == "interleaved") if rd else ops.NO_ROTATION
    ops.rope_cache_write(qkv, rotation, positions, seq_ids, table_d, q, pages_a, **kw)
    want = torch.zeros_like(q)
    ops.attention_decode(q, want, pages_a, table_d, kv_len, scratch, scale=hd ** -0.5, window=window,
                         pages_per_split=per, num_splits=n_splits, **kw)

    pages_b = pages.to(dev).clone()
    got = torch.full_like(q, 3.0)
    counters = torch.zeros(ops.decode_groups(B, H, G), dtype=torch.int32, device=dev)
    for _ in range(2):                       # twice: the share counters must be back at zero
        ops.attention_decode_fused(qkv, rotation, got, pages_b, table_d, kv_len, scratch, counters, write_kv=True,
                                   scale=hd ** -0.5, window=window, pages_per_split=per, num_splits=n_splits, **kw)
    assert int(counters.abs().sum()) == 0
    torch.cuda.synchronize()
    assert torch.equal(pages_a, pages_b)                      # the same keys and values were stored
    assert float((got.float() - want.float()).abs().max()) <= 2e-2


@pytest.mark.parametrize("H,G,hd", [(8, 2, 64), (4, 1, 128)])
def test_fused_decode_over_more_than_32_pages_in_one_share(H, G, hd):
    """One share per sequence holding 33 to 47 pages: the kernel that brings its pages by TMA keeps 32 entries
    of the page table in the first warp's lanes and has to fetch the next 32 on the way. Against the separate
    rotation and decode kernels (16-byte copies), on pages that are scattered over the cache."""
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    lengths = [2500, 2049, 3000, 70, 2113]
    B = len(lengths)
    _, pages, table = build_cache(lengths, G, hd, torch.bfloat16, seed=hd)
    g = torch.Generator().manual_seed(8)
    qkv = torch.randn(B, (H + 2 * G) * hd, generator=g).to(dev)
    rd = hd
    inv = (torch.rand(rd // 2, generator=g) * 0.01).to(dev)
    table_d = table.to(dev)
    kv_len = torch.tensor(lengths, dtype=torch.int32, device=dev)
    positions = kv_len - 1
    seq_ids = torch.arange(B, dtype=torch.int32, device=dev)
    kw = dict(num_heads=H, num_kv_heads=G, head_dim=hd)
    per = table.shape[1]

    def scratch(name, shape, dt):
        return torch.full(shape, float("nan"), dtype=dt, device=dev)

    rotation = ops.Rotation(inv, rd, False)
    pages_a = pages.to(dev).clone()
    q = torch.empty(B, H * hd, dtype=torch.bfloat16, device=dev)
    ops.rope_cache_write(qkv, rotation, positions, seq_ids, table_d, q, pages_a, **kw)
    want = torch.zeros_like(q)
    ops.attention_decode(q, want, pages_a, table_d, kv_len, scratch, scale=hd ** -0.5, window=None,
                         pages_per_split=per, num_splits=1, **kw)
    pages_b = pages.to(dev).clone()
    got = torch.full_like(q, 3.0)
    counters = torch.zeros(ops.decode_groups(B, H, G), dtype=torch.int32, device=dev)
    ops.attention_decode_fused(qkv, rotation, got, pages_b, table_d, kv_len, scratch, counters, write_kv=True,
                               scale=hd ** -0.5, window=None, pages_per_split=per, num_splits=1, **kw)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    assert torch.equal(pages_a, pages_b)
    assert float((got.float() - want.float()).abs().max()) <= 2e-2
