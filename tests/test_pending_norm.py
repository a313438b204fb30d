"""The hand-over of a norm that has not been computed yet (parts/base.py: PendingNorm): the block's
side of the protocol, without a GPU."""
import torch

from llmplayer_b200.parts.base import PendingNorm


class _Norm:
    fusable_rms = True


def test_materialises_once_and_keeps_source_and_norm():
    calls = []
    source = torch.arange(6.0).view(2, 3)
    out = torch.zeros(2, 3)

    def run():
        calls.append(1)
        out.copy_(source * 2)
        return out

    norm = _Norm()
    p = PendingNorm(source, norm, run)
    assert p.source is source and p.norm is norm and p.fusable
    assert not calls                          # nothing ran yet: a part may still apply the norm itself
    assert p.tensor() is out and p.tensor() is out
    assert len(calls) == 1
    assert torch.equal(out, source * 2)


def test_a_norm_that_cannot_be_fused_says_so():
    class Other:
        pass
    assert not PendingNorm(torch.zeros(1, 1), Other(), lambda: torch.zeros(1, 1)).fusable


def test_block_hands_pending_norm_only_to_parts_that_ask_for_it():
    """A block asks `takes_pending_norm` of its parts; a part that does not declare it gets the tensor."""
    from llmplayer_b200.parts.attention import Attention
    from llmplayer_b200.parts.feedforward import SwiGLU
    assert Attention.takes_pending_norm and SwiGLU.takes_pending_norm

    class Plain:
        pass
    assert not getattr(Plain(), "takes_pending_norm", False)


def test_buffers_kept_zero_are_restored_after_a_broken_step():
    from llmplayer_b200.engine.step import Workspace
    ws = Workspace("cpu")
    a = ws.get_zeroed("sums", 10)
    assert float(a.abs().sum()) == 0.0
    a += 3.0                                   # a step left partial sums behind
    other = ws.get("plain", (4,), torch.float32)
    other.fill_(7.0)
    ws.restore_zeroes()
    assert float(ws.get_zeroed("sums", 10).abs().sum()) == 0.0
    assert float(other.sum()) == 28.0          # ordinary scratch is left alone
    bigger = ws.get_zeroed("sums", 100)        # growing hands out zeroes again
    assert bigger.numel() == 100 and float(bigger.abs().sum()) == 0.0
