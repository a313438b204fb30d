"""A wait inside a tensor-core kernel that runs out: the kernel must return by itself, report through the
status word, and leave the engine usable.

Every wait on an mbarrier in the tcgen05 kernels is bounded. Here the loader of one launch is told (a test hook
of the library, ``lp_gemm_withhold_next``) never to bring one k-block: the waits for it give up after their
limit, each role records a code, the CTAs wind down (copies in flight awaited, tensor memory freed) and the kernel
ends. Nothing faults, traps or hangs. The host then finds the code (``KernelError``), restores what must be zero
between steps, and the next steps are correct. The reference's counterpart is its catch-and-fall-back after a
failed GPU call (inference/InferenceEngine.java:355-365)."""
import pytest
import torch

from helpers import TINY, assert_close, make_model, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def withhold_next(kblock):
    from llmplayer_b200.kernels import ops
    lib = ops.library("gemm_tcgen05")
    lib.lp_gemm_withhold_next.argtypes = [__import__("ctypes").c_int]
    assert lib.lp_gemm_withhold_next(int(kblock)) == 0


@pytest.mark.parametrize("mode", ["store", "accumulate"])
def test_a_product_whose_wait_runs_out_reports_and_returns(mode):
    from llmplayer_b200.errors import KernelError
    from llmplayer_b200.kernels import ops
    dev = "cuda:0"
    torch.manual_seed(3)
    M, N, K = 40, 384, 512                                   # a 64-token tile, eight k-blocks
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    code = ops.ACCUMULATE if mode == "accumulate" else ops.STORE
    ops.check_kernel_status()
    before = torch.full((M, N), 2.0, device=dev)
    out = before.clone()
    withhold_next(3)
    ops.gemm(a, w, out, code, splits=1)
    torch.cuda.synchronize()                                 # the kernel came back by itself
    with pytest.raises(KernelError, match="gave up waiting"):
        ops.check_kernel_status()
    assert torch.equal(out, before)                          # a CTA that gave up writes nothing
    ops.check_kernel_status()                                # the word was cleared by the report
    # the next launch is an ordinary one
    ref = a.double() @ w.double().T + (before.double() if mode == "accumulate" else 0)
    ops.gemm(a, w, out, code, splits=1)
    torch.cuda.synchronize()
    ops.check_kernel_status()
    assert float((out.double() - ref).abs().max() / ref.abs().max()) < 1e-5


def test_the_engine_goes_on_after_a_step_whose_kernel_gave_up(tmp_path):
    """Twenty sequences decode together (products with a 32-token tile on the tcgen05 kernel). One step's first
    such product gives up: ``check`` raises, the buffers and counters that are zero between uses are zero again,
    and new sequences on the same engine (same slots, same pages) get correct logits."""
    from llmplayer_b200 import Engine
    from llmplayer_b200.errors import KernelError
    model_dir = make_model(tmp_path, "D", dtype="bfloat16")
    vocab = TINY["D"][0]["vocab_size"]
    eng = Engine.load(model_dir, dtype="bfloat16", max_tokens=20 * 128, max_slots=20)
    seqs = [random_tokens(30 + 3 * i, vocab, seed=900 + i) for i in range(20)]

    def run_batch(withhold_at=None):
        slots = [eng.acquire() for _ in seqs]
        eng.step([(s, q[:-3]) for s, q in zip(slots, seqs)], [[] for _ in seqs])
        rows = []
        for k in (3, 2, 1):
            if withhold_at == k:
                withhold_next(1)
            rows.append(eng.step([(s, [q[-k]]) for s, q in zip(slots, seqs)], [[0]] * len(seqs)).cpu().clone())
        return slots, rows

    # the first decode step of a shape runs directly (later ones replay a captured graph, into which a hook that
    # acts on "the next launch" must not be recorded)
    slots, _ = run_batch(withhold_at=3)
    with pytest.raises(KernelError, match="gave up waiting"):
        eng.check()
    for key in eng.workspace._kept_zero:                     # partial-sum buffers and counters are zero again
        assert float(eng.workspace._buffers[key].float().abs().sum()) == 0.0, key
    for s in slots:
        eng.release(s)
    slots, rows = run_batch()
    eng.check()
    for i, q in enumerate(seqs):
        got = torch.stack([r[i] for r in rows])
        assert_close(got, plain_logits(model_dir, q)[-3:], "bfloat16", f"after a kernel gave up, request {i}", config="D")
    for s in slots:
        eng.release(s)
