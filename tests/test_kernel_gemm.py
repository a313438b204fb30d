"""The matrix-product kernels alone, against a float32 product of the same inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference(a, w, mode, out0=None):
    from llmplayer_b200.kernels import ops
    a32, w32 = a.double(), w.double()
    if mode == ops.SWIGLU:
        F = w.shape[0] // 2
        g, u = a32 @ w32[:F].T, a32 @ w32[F:].T
        return (g / (1 + torch.exp(-g))) * u
    r = a32 @ w32.T
    return r + out0.double() if mode == ops.ACCUMULATE else r


def rel_err(got, ref):
    return float((got.double() - ref).abs().max() / ref.abs().max())


SHAPES = [(1, 64, 64), (5, 100, 72), (8, 3072, 2048), (17, 130, 200), (64, 256, 4096), (70, 264, 136),
          (300, 520, 328), (1, 128256, 64), (513, 640, 1024), (2048, 392, 264), (777, 3000, 136)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("mode", ["store", "accumulate", "swiglu"])
def test_tensor_core_gemm(M, N, K, mode):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(M * 7 + N + K)
    dev = "cuda:0"
    code = {"store": ops.STORE, "accumulate": ops.ACCUMULATE, "swiglu": ops.SWIGLU}[mode]
    if mode == "swiglu" and N > 4096:
        pytest.skip("no gated product that wide")
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N * (2 if mode == "swiglu" else 1), K, device=dev) / K ** 0.5).to(torch.bfloat16)
    w_kernel = ops.interleave_gate_up(w[:N], w[N:]) if mode == "swiglu" else w
    for out_dtype in ([torch.float32] if mode == "accumulate" else [torch.float32, torch.bfloat16]):
        out0 = torch.randn(M, N, device=dev)
        out = out0.clone().to(out_dtype)
        ops.gemm(a, w_kernel, out, code)
        torch.cuda.synchronize()
        ops.check_kernel_status()
        ref = reference(a, w, code, out0)
        tol = 1e-5 if out_dtype == torch.float32 else 5e-3          # bf16 output: one rounding
        assert rel_err(out, ref) < tol, (M, N, K, mode, out_dtype, rel_err(out, ref))


@pytest.mark.parametrize("tile", [16, 32, 64, 128, 256])
def test_gated_epilogue_at_every_tile(tile):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(tile)
    M, F, K = 300, 264, 520
    a = torch.randn(M, K, device="cuda:0").to(torch.bfloat16)
    w = (torch.randn(2 * F, K, device="cuda:0") / K ** 0.5).to(torch.bfloat16)
    out = torch.full((M, F), 7.0, device="cuda:0", dtype=torch.bfloat16)
    ops.gemm(a, ops.interleave_gate_up(w[:F], w[F:]), out, ops.SWIGLU, block_tok=tile)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    assert rel_err(out, reference(a, w, ops.SWIGLU)) < 5e-3


@pytest.mark.parametrize("tile,splits", [(16, 1), (16, 4), (32, 3), (64, 2), (128, 1), (256, 1), (256, 2)])
def test_every_tile_and_split(tile, splits):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(tile + splits)
    M, N, K = 333, 392, 1096
    a = torch.randn(M, K, device="cuda:0").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda:0") / K ** 0.5).to(torch.bfloat16)
    out = torch.full((M, N), 7.0, device="cuda:0")
    ops.gemm(a, w, out, ops.STORE, block_tok=tile, splits=splits)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    assert rel_err(out, reference(a, w, ops.STORE)) < 1e-5


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 100, 70), (64, 256, 513), (130, 70, 33)])
@pytest.mark.parametrize("mode", ["store", "accumulate", "swiglu"])
@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.bfloat16, torch.float32)])
def test_plain_gemm(M, N, K, mode, dtypes):
    from llmplayer_b200.kernels import ops
    torch.manual_seed(M + N + K)
    code = {"store": ops.STORE, "accumulate": ops.ACCUMULATE, "swiglu": ops.SWIGLU}[mode]
    a = torch.randn(M, K, device="cuda:0").to(dtypes[0])
    w = (torch.randn(N * (2 if mode == "swiglu" else 1), K, device="cuda:0") / K ** 0.5).to(dtypes[1])
    out0 = torch.randn(M, N, device="cuda:0")
    out = out0.clone()
    ops.gemm_plain(a, w, out, code)
    assert rel_err(out, reference(a, w, code, out0)) < 2e-6


def test_plain_gemm_rows_do_not_depend_on_the_batch():
    from llmplayer_b200.kernels import ops
    a = torch.randn(70, 300, device="cuda:0")
    w = torch.randn(90, 300, device="cuda:0")
    whole = torch.empty(70, 90, device="cuda:0")
    ops.gemm_plain(a, w, whole)
    one = torch.empty(1, 90, device="cuda:0")
    ops.gemm_plain(a[37:38].contiguous(), w, one)
    assert torch.equal(whole[37:38], one)


def test_refusals():
    from llmplayer_b200.errors import KernelError
    from llmplayer_b200.kernels import ops
    a = torch.randn(4, 20, device="cuda:0").to(torch.bfloat16)
    w = torch.randn(8, 20, device="cuda:0").to(torch.bfloat16)
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm(a, w, torch.empty(4, 8, device="cuda:0"))
    with pytest.raises(KernelError, match="gemm"):
        ops.gemm(a, w, torch.empty(4, 9, device="cuda:0"))
    with pytest.raises(KernelError):
        ops.gemm_plain(a.cpu(), w, torch.empty(4, 8, device="cuda:0"))


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (4, 2048, 8192), (2, 640, 328), (4, 128, 200), (3, 3072, 512)])
def test_accumulate_with_the_following_norm(M, N, K):
    """The product adds into the residual rows; its last CTA then writes their RMS norm and
    clears a buffer. Twice in a row: the CTA counter must be back at zero."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(N + K)
    dev = "cuda:0"
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    gain = (1 + 0.1 * torch.randn(N, device=dev))
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    for _ in range(2):
        out0 = torch.randn(M, N, device=dev)
        out = out0.clone()
        normed = torch.full((M, N), 9.0, device=dev, dtype=torch.bfloat16)
        junk = torch.full((3000,), 4.0, device=dev)
        ops.gemm(a, w, out, ops.ACCUMULATE, norm_after=(gain, 1e-5, normed, junk, counter))
        torch.cuda.synchronize()
        ops.check_kernel_status()
        ref = reference(a, w, ops.ACCUMULATE, out0)
        assert rel_err(out, ref) < 1e-5
        want = ref * torch.rsqrt((ref * ref).mean(dim=1, keepdim=True) + 1e-5) * gain.double()
        assert rel_err(normed, want) < 8e-3                  # one bfloat16 rounding
        assert float(junk.abs().sum()) == 0.0


# --------------------------------------------------------------------------- a handful of tokens
FEW_SHAPES = [(1, 64, 64), (3, 200, 72), (8, 3072, 2048), (9, 130, 200), (16, 520, 328), (5, 96, 1000),
              (33, 200, 136), (64, 264, 520), (24, 2048, 2048)]


@pytest.mark.parametrize("M,N,K", FEW_SHAPES)
@pytest.mark.parametrize("mode", ["store", "accumulate", "swiglu"])
def test_few_token_product(M, N, K, mode):
    """The products for at most 64 rows with bfloat16 activations (the mma.sync kernel up to 16 rows, the one-tile
    tcgen05 kernel beyond), against a float64 product."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(M * 11 + N + K)
    dev = "cuda:0"
    code = {"store": ops.STORE, "accumulate": ops.ACCUMULATE, "swiglu": ops.SWIGLU}[mode]
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N * (2 if mode == "swiglu" else 1), K, device=dev) / K ** 0.5).to(torch.bfloat16)
    w_kernel = ops.interleave_gate_up(w[:N], w[N:]) if mode == "swiglu" else w
    out0 = torch.randn(M, N, device=dev) if mode == "accumulate" else torch.zeros(M, N, device=dev)
    out = out0.clone()
    side = torch.full((37,), 3.0, device=dev)
    ops.gemm_few(a, w_kernel, out, code, zero=side)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    assert rel_err(out, reference(a, w, code, out0)) < 1e-5
    assert float(side.abs().max()) == 0.0, "the buffer to clear on the side was not cleared"


@pytest.mark.parametrize("M,N,K", FEW_SHAPES)
@pytest.mark.parametrize("mode", ["store", "swiglu"])
def test_few_token_product_applies_the_norm(M, N, K, mode):
    """x float32 -> RMS norm (gain, eps) -> product, in one kernel: either the kernel applies the row
    factor itself, or (K shared out over CTAs) it reports the rows' sums of squares instead."""
    from llmplayer_b200.kernels import ops
    torch.manual_seed(M * 13 + N + K)
    dev = "cuda:0"
    code = {"store": ops.STORE, "swiglu": ops.SWIGLU}[mode]
    eps = 3e-6
    x = torch.randn(M, K, device=dev) * 3.0
    x[0, 5 % K] = 40.0                                  # a row whose factor differs clearly from the others'
    gain = 1.0 + 0.3 * torch.randn(K, device=dev)
    w = (torch.randn(N * (2 if mode == "swiglu" else 1), K, device=dev) / K ** 0.5).to(torch.bfloat16)
    w_kernel = ops.interleave_gate_up(w[:N], w[N:]) if mode == "swiglu" else w
    out = torch.zeros(M, N, device=dev)
    sumsq = torch.zeros(64, device=dev)
    deferred = ops.gemm_few(x, w_kernel, out, code, norm=(gain, eps), sumsq=sumsq)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    xd = x.double()
    factor = 1.0 / torch.sqrt((xd * xd).mean(dim=1, keepdim=True) + eps)
    # the kernel rounds x * gain to bfloat16 and applies the row factor in float32 afterwards
    operand = (x * gain).to(torch.bfloat16)
    ref = reference(operand, w, code) if mode == "store" else None
    if mode == "store":
        if deferred:
            assert rel_err(sumsq[:M], (xd * xd).sum(dim=1)) < 1e-5
            got = out.double() * factor
        else:
            got = out.double()
        assert rel_err(got, ref * factor) < 1e-5
    else:
        assert not deferred
        F = N
        g = (operand.double() @ w.double()[:F].T) * factor
        u = (operand.double() @ w.double()[F:].T) * factor
        assert rel_err(out, (g / (1 + torch.exp(-g))) * u) < 1e-5
    # and against the norm as the model defines it (rounding of the normed row to bfloat16 differs slightly)
    normed = (xd * factor * gain.double())
    full = reference(normed.float().to(torch.bfloat16), w, code)
    got = out.double() * factor if deferred else out.double()
    assert rel_err(got, full) < 2e-2


@pytest.mark.parametrize("H,G,hd,pairing,rotary", [(32, 8, 64, "split_half", True), (6, 4, 64, "split_half", True),
                                                   (24, 8, 128, "split_half", True), (5, 3, 128, "interleaved", True),
                                                   (3, 1, 256, "split_half", True), (7, 2, 32, "interleaved", True),
                                                   (4, 2, 64, "split_half", False)])
@pytest.mark.parametrize("shares_kv", [False, True])
def test_projection_with_rotation_and_cache_write_in_its_epilogue(H, G, hd, pairing, rotary, shares_kv):
    """The fused q|k|v projection of a long step against the separate kernels: the float32 product, then the
    rotation kernel that writes queries and the cache. Two sequences of unequal lengths, the second continued
    at a position in the middle of a page, pages scattered."""
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    torch.manual_seed(H * 100 + hd)
    K = 328
    lengths, starts = [700, 333], [0, 41]                       # new tokens and first positions of the two sequences
    T = sum(lengths)
    heads = H if shares_kv else H + 2 * G
    x = torch.randn(T, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(heads * hd, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lengths)]).to(torch.int32).to(dev)
    seq_ids = torch.cat([torch.full((n,), i) for i, n in enumerate(lengths)]).to(torch.int32).to(dev)
    width = max(-(-(s + n) // 64) for s, n in zip(starts, lengths))
    num_pages = 2 * width + 3
    order = torch.randperm(num_pages)[:2 * width].reshape(2, width).to(torch.int32).to(dev)
    rd = hd if rotary else 0
    inv = (torch.rand(max(rd // 2, 1), device=dev) * 0.3) if rd else None
    rotation = ops.Rotation(inv, rd, pairing == "interleaved") if rd else ops.NO_ROTATION
    assert ops.qkv_rope_serves(rotation, hd)

    def fresh_pages():
        return torch.full((num_pages, 2, G, 64, hd), 5.0, device=dev, dtype=torch.bfloat16)

    # separate kernels
    qkv = torch.empty(T, heads * hd, device=dev)
    ops.gemm(x, w, qkv, ops.STORE)
    q_ref = torch.empty(T, H * hd, device=dev, dtype=torch.bfloat16)
    pages_ref = fresh_pages()
    ops.rope_cache_write(qkv, rotation, positions, seq_ids, order, q_ref, None if shares_kv else pages_ref,
                         num_heads=H, num_kv_heads=G, head_dim=hd)
    # fused
    q_got = torch.full_like(q_ref, 9.0)
    pages_got = fresh_pages()
    angles = None
    if rd:
        angles = torch.empty(T, rd // 2, 2, device=dev)
        ops.rope_angles(positions, rotation, angles)
    ops.gemm_qkv_rope(x, w, angles, pairing == "interleaved", positions, seq_ids, order, q_got,
                      None if shares_kv else pages_got, num_heads=H, num_kv_heads=G, head_dim=hd)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    scale = float(q_ref.float().abs().max())
    assert float((q_got.float() - q_ref.float()).abs().max()) <= 8e-3 * scale        # one bfloat16 rounding apart at most
    if not shares_kv:
        assert float((pages_got.float() - pages_ref.float()).abs().max()) <= 8e-3 * max(scale, 5.0)
        untouched = pages_ref == 5.0
        assert torch.equal(pages_got[untouched], pages_ref[untouched])              # nothing written beside the tokens' rows
    else:
        assert torch.equal(pages_got, fresh_pages())
