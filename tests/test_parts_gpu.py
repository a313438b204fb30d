"""Each part alone, built from its specification, against the plain functions."""
import math
import zlib

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
# The cache keeps keys and values, and the attention kernels take queries, in the activation type. With
# queries and keys made large on purpose (sharp attention shows a wrong key), that one rounding alone moves a
# bfloat16 result by 1-2 % of its largest value, so the plain attention below rounds the same three tensors.
STORED = {"float32": None, "bfloat16": torch.bfloat16}
# ... and a block hands its parts the normed stream in the activation type.
ACTIVATION = {"float32": None, "bfloat16": torch.bfloat16}


def kept_as(t, dtype):
    """``t`` after a round trip through ``dtype`` (None: unchanged)."""
    return t if dtype is None else t.to(dtype).to(t.dtype)


@pytest.fixture(autouse=True)
def own_random_numbers(request):
    """Every test draws from its own seed, so that no result depends on which tests ran before it."""
    torch.manual_seed(zlib.crc32(request.node.name.encode()))


def runtime(dtype):
    from llmplayer_b200.parts.base import Runtime
    return Runtime(device=torch.device(DEV), dtype=dtype)


def rel(got, ref):
    return float((got.double().cpu() - ref.double()).abs().max() / ref.double().abs().max())


def make_context(cache, workspace, slots, new_tokens):
    """A step for ``slots`` bringing ``new_tokens[i]`` tokens each (token ids do not matter here)."""
    from llmplayer_b200.engine.step import SequenceStep, StepContext
    cache.reserve(slots, new_tokens)
    seqs, start = [], 0
    for s, n in zip(slots, new_tokens):
        seqs.append(SequenceStep(s, start, n, cache.length(s)))
        start += n
    return StepContext(workspace, seqs, [0] * start, cache.page_tables(slots), [])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [100, 2048, 5000])
def test_rms_norm_part(dtype, d):
    from llmplayer_b200.parts import NORMS
    from llmplayer_b200.parts.specs import NormSpec
    rt = runtime(dtype)
    part = NORMS.build(NormSpec(size=d, eps=3e-6, weight="w"))
    assert part.tensor_specs()["w"].shape == (d,)
    w = 1 + 0.1 * torch.randn(d)
    part.load({"w": w.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32)}, rt)
    x = torch.randn(7, d) * 3
    w_used = part.weight.cpu()
    out = torch.empty(7, d, device=DEV, dtype=rt.act_dtype)
    part.apply(x.to(DEV), out)
    assert rel(out, P.rms_norm(x.double(), w_used.double(), 3e-6)) < TOL[dtype]
    # chosen rows, the fused residual add, and a buffer cleared on the side
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    some = torch.empty(3, d, device=DEV, dtype=rt.act_dtype)
    part.apply(x.to(DEV), some, rows=rows)
    assert rel(some, P.rms_norm(x[[5, 0, 5]].double(), w_used.double(), 3e-6)) < TOL[dtype]
    add = torch.randn(7, d)
    xd = x.to(DEV).clone()
    junk = torch.full((1000,), 5.0, device=DEV)
    part.apply(xd, out, add=add.to(DEV), clear=junk)
    assert torch.allclose(xd.cpu(), x + add, atol=1e-6)
    assert rel(out, P.rms_norm((x + add).double(), w_used.double(), 3e-6)) < TOL[dtype]
    assert float(junk.abs().sum()) == 0.0


@pytest.mark.parametrize("pairing", ["split_half", "interleaved"])
@pytest.mark.parametrize("hd,rd", [(16, 16), (48, 32), (128, 128)])
def test_rotation_and_cache_write(pairing, hd, rd):
    from llmplayer_b200.cache import KVRequest, SequenceCache
    from llmplayer_b200.engine.step import Workspace
    from llmplayer_b200.kernels import ops
    from llmplayer_b200.parts import POSITIONS
    from llmplayer_b200.parts.specs import PositionSpec
    H, G = 3, 2
    rope = POSITIONS.build(PositionSpec(kind="rope", head_dim=hd, rotary_dim=rd, theta=777.0, pairing=pairing))
    rope.load({}, runtime("float32"))
    cache = SequenceCache([KVRequest(G, hd)], max_tokens=512, max_slots=3, kv_dtype=torch.float32, device=DEV)
    ws = Workspace(DEV)
    a, b = cache.acquire(), cache.acquire()
    ctx = make_context(cache, ws, [a, b], [70, 5])          # crosses a page boundary
    cache.commit([a, b], [70, 5])
    ctx2 = make_context(cache, ws, [b], [3])                # continues b at position 5
    T = 3
    qkv = torch.randn(T, (H + 2 * G) * hd)
    q_out = torch.empty(T, H * hd, device=DEV)
    view = cache.view(0)
    ops.rope_cache_write(qkv.to(DEV), rope.rotation(), ctx2.positions, ctx2.seq_ids, ctx2.page_tables[0], q_out,
                         view.pages, num_heads=H, num_kv_heads=G, head_dim=hd)
    pos = torch.tensor([5, 6, 7])
    inv = P.rope_inverse_frequencies(rd, 777.0)
    q_ref = P.rope_rotate(qkv[:, :H * hd].reshape(T, H, hd).double(), pos, inv, pairing)
    k_ref = P.rope_rotate(qkv[:, H * hd:(H + G) * hd].reshape(T, G, hd).double(), pos, inv, pairing)
    v_ref = qkv[:, (H + G) * hd:].reshape(T, G, hd).double()
    assert rel(q_out.reshape(T, H, hd), q_ref) < 1e-6
    page = cache.page_tables([b])[0][0][0]
    stored = view.pages[page].cpu()                         # [2, G, 64, hd]
    assert rel(stored[0, :, 5:8].transpose(0, 1), k_ref) < 1e-6
    assert rel(stored[1, :, 5:8].transpose(0, 1), v_ref) < 1e-6
    assert float(stored[:, :, 8:].abs().sum()) == 0.0       # nothing else was touched
    assert torch.equal(q_ref[..., rd:], qkv[:, :H * hd].reshape(T, H, hd).double()[..., rd:])   # partial rotation


def attention_tensors(d, H, G, hd, seed):
    g = torch.Generator().manual_seed(seed)
    s = 1.0 / math.sqrt(d)
    return {"q": torch.randn(H * hd, d, generator=g) * s * 3, "k": torch.randn(G * hd, d, generator=g) * s * 3,
            "v": torch.randn(G * hd, d, generator=g) * s, "o": torch.randn(d, H * hd, generator=g) * s}


def plain_attention_part(x, w, H, G, hd, theta, positions, window, stored=None):
    T = x.shape[0]
    inv = P.rope_inverse_frequencies(hd, theta)
    q = P.rope_rotate((x @ w["q"].T).reshape(T, H, hd), positions, inv)
    k = P.rope_rotate((x @ w["k"].T).reshape(T, G, hd), positions, inv)
    v = (x @ w["v"].T).reshape(T, G, hd)
    if stored is not None:
        q, k, v = (t.to(stored).to(x.dtype) for t in (q, k, v))
    return P.attention(q, k, v, 1.0 / math.sqrt(hd), window=window, q_positions=positions).reshape(T, H * hd) @ w["o"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,window", [(4, 2, 16, None), (6, 1, 32, 20), (3, 3, 64, 70)])
def test_attention_part_in_steps(dtype, H, G, hd, window):
    """One attention layer alone: a prompt, then a chunk, then single tokens; every output must
    equal the whole-sequence plain attention (so the window's edge and the cache are exercised)."""
    from llmplayer_b200.cache import SequenceCache
    from llmplayer_b200.engine.step import Workspace
    from llmplayer_b200.parts import MIXERS
    from llmplayer_b200.parts.specs import AttentionSpec, PositionSpec
    d, T = 72, 150
    rt = runtime(dtype)
    spec = AttentionSpec(hidden_size=d, num_heads=H, num_kv_heads=G, head_dim=hd, scale=1.0 / math.sqrt(hd),
                         position=PositionSpec(kind="rope", head_dim=hd, rotary_dim=hd, theta=5000.0),
                         q="q", k="k", v="v", o="o", window=window)
    part = MIXERS.build(spec)
    assert set(part.tensor_specs()) == {"q", "k", "v", "o"}
    w = attention_tensors(d, H, G, hd, seed=H)
    held = {n: t.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32) for n, t in w.items()}
    part.load(held, rt)
    cache = SequenceCache([part.cache_request()], max_tokens=256, max_slots=2, kv_dtype=rt.kv_dtype, device=DEV)
    ws = Workspace(DEV)
    x = torch.randn(T, d).to(rt.act_dtype)
    ref = plain_attention_part(x.double(), {n: t.double() for n, t in held.items()}, H, G, hd, 5000.0,
                               torch.arange(T), window, stored=STORED[dtype])
    slot = cache.acquire()
    got = []
    for n in [90, 30] + [1] * 30:
        ctx = make_context(cache, ws, [slot], [n])
        start = cache.length(slot)
        residual = torch.zeros(n, d, device=DEV)
        part.forward(ctx, cache.view(0), x[start:start + n].to(DEV).contiguous(), residual)
        cache.commit([slot], [n])
        got.append(residual.cpu())
    assert rel(torch.cat(got), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,F,T", [(72, 200, 5), (256, 1000, 70), (2048, 8192, 8)])
def test_swiglu_part(dtype, d, F, T):
    from llmplayer_b200.engine.step import StepContext, Workspace
    from llmplayer_b200.parts import FEED_FORWARDS
    from llmplayer_b200.parts.specs import SwiGLUSpec
    rt = runtime(dtype)
    part = FEED_FORWARDS.build(SwiGLUSpec(hidden_size=d, intermediate_size=F, gate="g", up="u", down="d"))
    g = torch.Generator().manual_seed(d)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    w = {"g": (torch.randn(F, d, generator=g) / d ** 0.5).to(store), "u": (torch.randn(F, d, generator=g) / d ** 0.5).to(store),
         "d": (torch.randn(d, F, generator=g) / F ** 0.5).to(store)}
    part.load(w, rt)
    x = torch.randn(T, d, generator=g).to(rt.act_dtype)
    ctx = StepContext(Workspace(DEV), [], [0] * T, [], [])
    residual0 = torch.randn(T, d, generator=g)
    residual = residual0.to(DEV).clone()
    part.forward(ctx, x.to(DEV), residual)
    ref = residual0.double() + P.swiglu(x.double(), w["g"].double(), w["u"].double(), w["d"].double())
    assert rel(residual, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head(dtype, tied):
    from llmplayer_b200.engine.step import StepContext, Workspace
    from llmplayer_b200.parts.embedding import Embedding, LinearHead
    from llmplayer_b200.parts.specs import EmbeddingSpec, HeadSpec, NormSpec
    V, d = 301, 88
    rt = runtime(dtype)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = {"emb": (torch.randn(V, d) * 0.3).to(store), "norm": (1 + 0.1 * torch.randn(d)).to(store),
               "head": (torch.randn(V, d) * 0.3).to(store)}
    emb = Embedding(EmbeddingSpec(V, d, "emb"))
    head = LinearHead(HeadSpec(V, d, NormSpec(d, 1e-5, "norm"), "emb" if tied else "head"))
    emb.load(tensors, rt)
    head.load(tensors, rt)
    if tied:
        assert emb.table.data_ptr() == head.proj.weight.data_ptr()          # one table on the device
    tokens = torch.tensor([5, 300, 0, 17], dtype=torch.int32, device=DEV)
    x = torch.empty(4, d, device=DEV)
    emb.forward(tokens, x)
    assert torch.equal(x.cpu(), tensors["emb"].float()[[5, 300, 0, 17]])   # no scaling
    ctx = StepContext(Workspace(DEV), [], [0] * 4, [], [])
    rows = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    logits = torch.empty(2, V, device=DEV)
    head.forward(ctx, x, rows, logits)
    hw = tensors["emb" if tied else "head"].double()
    ref = P.rms_norm(x.cpu().double()[[3, 1]], tensors["norm"].double(), 1e-5) @ hw.T
    assert rel(logits, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part(dtype):
    from llmplayer_b200.cache import SequenceCache
    from llmplayer_b200.engine.step import Workspace
    from llmplayer_b200.parts import BLOCKS
    from llmplayer_b200.parts.specs import AttentionSpec, BlockSpec, NormSpec, PositionSpec, SwiGLUSpec
    d, H, G, hd, F, T = 96, 4, 2, 32, 200, 40
    rt = runtime(dtype)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    spec = BlockSpec(
        mixer_norm=NormSpec(d, 1e-5, "n1"),
        mixer=AttentionSpec(d, H, G, hd, 1.0 / math.sqrt(hd), PositionSpec("rope", hd, hd, 10000.0), q="q", k="k",
                            v="v", o="o"),
        ffn_norm=NormSpec(d, 1e-5, "n2"), ffn=SwiGLUSpec(d, F, "g", "u", "dn"))
    block = BLOCKS.build(spec)
    w = attention_tensors(d, H, G, hd, seed=9)
    w.update({"n1": 1 + 0.1 * torch.randn(d), "n2": 1 + 0.1 * torch.randn(d), "g": torch.randn(F, d) / d ** 0.5,
              "u": torch.randn(F, d) / d ** 0.5, "dn": torch.randn(d, F) / F ** 0.5})
    assert set(block.tensor_specs()) == set(w)
    held = {n: t.to(store) for n, t in w.items()}
    block.load(held, rt)
    cache = SequenceCache([block.cache_request()], max_tokens=128, max_slots=1, kv_dtype=rt.kv_dtype, device=DEV)
    slot = cache.acquire()
    x0 = torch.randn(T, d)
    ctx = make_context(cache, Workspace(DEV), [slot], [T])
    x = x0.to(DEV).clone()
    block.forward(ctx, cache.view(0), x)
    hw = {n: t.double() for n, t in held.items()}
    r = x0.double()
    act = ACTIVATION[dtype]
    r = r + plain_attention_part(kept_as(P.rms_norm(r, hw["n1"], 1e-5), act), hw, H, G, hd, 10000.0, torch.arange(T),
                                 None, stored=STORED[dtype])
    r = r + P.swiglu(kept_as(P.rms_norm(r, hw["n2"], 1e-5), act), hw["g"], hw["u"], hw["dn"])
    assert rel(x, r) < TOL[dtype]


@pytest.mark.parametrize("hd,dtype", [(16, torch.float32), (64, torch.bfloat16), (48, torch.bfloat16)])
def test_rotation_and_cache_write_of_a_long_prompt(hd, dtype):
    """A prompt of some hundred tokens takes the kernel that works in fours (whole heads, split halves)."""
    from llmplayer_b200.cache import KVRequest, SequenceCache
    from llmplayer_b200.engine.step import Workspace
    from llmplayer_b200.kernels import ops
    from llmplayer_b200.parts import POSITIONS
    from llmplayer_b200.parts.specs import PositionSpec
    H, G, T = 5, 2, 333
    rope = POSITIONS.build(PositionSpec(kind="rope", head_dim=hd, rotary_dim=hd, theta=50000.0, pairing="split_half"))
    rope.load({}, runtime("float32"))
    cache = SequenceCache([KVRequest(G, hd)], max_tokens=1024, max_slots=2, kv_dtype=dtype, device=DEV)
    ws = Workspace(DEV)
    a = cache.acquire()
    ctx = make_context(cache, ws, [a], [T])
    qkv = torch.randn(T, (H + 2 * G) * hd, generator=torch.Generator().manual_seed(hd))
    q_out = torch.empty(T, H * hd, device=DEV, dtype=dtype)
    view = cache.view(0)
    ops.rope_cache_write(qkv.to(DEV), rope.rotation(), ctx.positions, ctx.seq_ids, ctx.page_tables[0], q_out,
                         view.pages, num_heads=H, num_kv_heads=G, head_dim=hd)
    pos = torch.arange(T)
    inv = P.rope_inverse_frequencies(hd, 50000.0)
    q_ref = P.rope_rotate(qkv[:, :H * hd].reshape(T, H, hd).double(), pos, inv, "split_half")
    k_ref = P.rope_rotate(qkv[:, H * hd:(H + G) * hd].reshape(T, G, hd).double(), pos, inv, "split_half")
    v_ref = qkv[:, (H + G) * hd:].reshape(T, G, hd).double()
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert rel(q_out.float().reshape(T, H, hd), q_ref) < tol
    table = cache.page_tables([a])[0][0]
    stored = torch.cat([view.pages[p].float().cpu() for p in table], dim=2)[:, :, :T]      # [2, G, T, hd]
    assert rel(stored[0].transpose(0, 1), k_ref) < tol
    assert rel(stored[1].transpose(0, 1), v_ref) < tol


@pytest.mark.parametrize("d,dtype", [(2048, torch.bfloat16), (264, torch.float32), (4096, torch.bfloat16)])
def test_rms_norm_of_rows_of_a_multiple_of_four(d, dtype):
    """Rows of a multiple of 4 values without a residual add take the kernel that loads four values at a time."""
    from llmplayer_b200.kernels import ops
    g = torch.Generator().manual_seed(d)
    x = (torch.randn(37, d, generator=g) * 3).to(DEV)
    w = (1 + 0.2 * torch.randn(d, generator=g)).to(DEV)
    out = torch.empty(37, d, device=DEV, dtype=dtype)
    junk = torch.full((1000,), 5.0, device=DEV)
    ops.rmsnorm(x, w, 3e-6, out, clear=junk)
    assert rel(out.float(), P.rms_norm(x.double().cpu(), w.double().cpu(), 3e-6)) < (1e-6 if dtype == torch.float32 else 1e-2)
    assert float(junk.abs().sum()) == 0.0
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=DEV)
    sel = torch.empty(3, d, device=DEV, dtype=dtype)
    ops.rmsnorm(x, w, 3e-6, sel, rows=rows)
    assert rel(sel.float(), P.rms_norm(x[rows.long()].double().cpu(), w.double().cpu(), 3e-6)) < (1e-6 if dtype == torch.float32 else 1e-2)

