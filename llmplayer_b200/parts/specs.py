"""Descriptions of the parts a decoder is put together from.

A specification is plain data: it carries every size, constant and tensor name
its part needs, and a ``kind`` that the part registries resolve to a class.
An architecture turns its configuration into a :class:`ModelLayout`; nothing
below that layout knows which architecture it came from.

The reference describes the same pieces by fields of one configuration object
(model/ModelConfig.java:100-156) and wires them in code
(inference/InferenceEngine.java:53-101, inference/TransformerBlock.java:64-159).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

# Kinds of tensors: they decide how random weights are drawn and how a tensor
# is held on the device.
MATRIX = "matrix"   # [out, in] weight of a linear map, or an embedding table
GAIN = "gain"       # per-feature multiplier of a norm, drawn around one
INTEGER = "integer"  # integer table, held as int32


@dataclass(frozen=True)
class TensorSpec:
    """Shape and kind of one named tensor of a model folder."""
    shape: Tuple[int, ...]
    kind: str = MATRIX


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    weight: str
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class Llama3Scaling:
    """Frequency-dependent stretching of rotary wavelengths ("llama3" rope_scaling)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position: int


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    ``kind="rope"`` rotates the first ``rotary_dim`` features of each head;
    ``pairing`` is ``"split_half"`` (feature i with i + rotary_dim/2) or
    ``"interleaved"`` (2i with 2i+1). ``kind="none"`` leaves them as they are.
    """
    kind: str = "rope"
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 0.0
    scaling: Optional[Llama3Scaling] = None
    pairing: str = "split_half"


@dataclass(frozen=True)
class AttentionSpec:
    """Softmax attention over the cached keys of a sequence, with grouped query heads.

    ``window`` limits a query at position p to keys at positions > p - window
    (None: all keys). ``shares_kv`` marks a layer that projects no keys or
    values and attends over the cache of the schedule entry it is pointed at.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: PositionSpec
    q: str
    o: str
    k: Optional[str] = None
    v: Optional[str] = None
    window: Optional[int] = None
    shares_kv: bool = False
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(silu(gate x) * (up x))."""
    hidden_size: int
    intermediate_size: int
    gate: str
    up: str
    down: str
    kind: str = "swiglu"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how its norms, mixer and feed-forward are arranged.

    ``kind="prenorm"``: x += mixer(norm(x)); x += feed_forward(norm(x)).
    """
    mixer_norm: NormSpec
    mixer: object
    ffn_norm: NormSpec
    ffn: object
    kind: str = "prenorm"


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    weight: str
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Final norm and projection to the vocabulary. ``weight`` may name the
    embedding table (a tied head)."""
    vocab_size: int
    hidden_size: int
    norm: NormSpec
    weight: str
    kind: str = "linear_head"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``reads_cache_of`` is the index of an earlier entry
    of the schedule whose cache this run attends over instead of keeping its own."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelLayout:
    embedding: EmbeddingSpec
    layers: Tuple[BlockSpec, ...]
    head: HeadSpec
    schedule: Tuple[ScheduleEntry, ...] = field(default=())

    def run_order(self) -> Tuple[ScheduleEntry, ...]:
        """The schedule, or every layer once in order when none is given."""
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i) for i in range(len(self.layers)))
