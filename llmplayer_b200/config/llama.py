"""Configuration of the dense pre-norm decoder ``LlamaForCausalLM``.

Keys are those of the architecture's own ``config.json``. The reference reads
the same quantities from GGUF metadata (model/ModelConfig.java:242-501):
block_count :249, embedding_length :248, head_count :250, head_count_kv :260
(default: head_count), key_length :319/:342-345 (default: width / heads),
feed_forward_length :271, rope.freq_base :288, layer_norm_rms_epsilon :289,
context_length :263. A tied head is the absence of ``output.weight`` there
(model/ModelLoader.java:207-214) and the flag ``tie_word_embeddings`` here.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from ..errors import ConfigError
from ..parts.specs import (
    AttentionSpec, BlockSpec, EmbeddingSpec, HeadSpec, Llama3Scaling, ModelLayout,
    NormSpec, PositionSpec, SwiGLUSpec,
)
from .registry import ArchitectureConfig, register_architecture

_MISSING = object()


def _get(raw: dict, key: str, kind, default=_MISSING):
    value = raw.get(key, _MISSING)
    if value is _MISSING or value is None:
        if default is _MISSING:
            raise ConfigError(f"config.json lacks the key {key!r}")
        return default
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"{key} must be an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{key} must be a number, got {value!r}")
        return float(value)
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"{key} must be true or false, got {value!r}")
        return value
    raise AssertionError(kind)


def _positive(name: str, value) -> None:
    if not value > 0:
        raise ConfigError(f"{name} must be positive, got {value!r}")


def _read_scaling(raw: dict) -> Optional[Llama3Scaling]:
    block = raw.get("rope_scaling")
    if block is None:
        block = raw.get("rope_parameters")
        if isinstance(block, dict) and block.get("rope_type", block.get("type", "default")) == "default":
            block = None
    if block is None:
        return None
    if not isinstance(block, dict):
        raise ConfigError("rope_scaling must be an object or null")
    rope_type = block.get("rope_type", block.get("type"))
    if rope_type in (None, "default"):
        return None
    if rope_type != "llama3":
        raise ConfigError(f"rope_scaling type {rope_type!r} is not supported (known: llama3, default)")
    scaling = Llama3Scaling(
        factor=_get(block, "factor", float),
        low_freq_factor=_get(block, "low_freq_factor", float),
        high_freq_factor=_get(block, "high_freq_factor", float),
        original_max_position=_get(block, "original_max_position_embeddings", int),
    )
    _positive("rope_scaling.factor", scaling.factor)
    _positive("rope_scaling.low_freq_factor", scaling.low_freq_factor)
    _positive("rope_scaling.original_max_position_embeddings", scaling.original_max_position)
    if not scaling.high_freq_factor > scaling.low_freq_factor:
        raise ConfigError("rope_scaling.high_freq_factor must exceed low_freq_factor")
    return scaling


def _read_token_ids(raw: dict, key: str) -> Tuple[int, ...]:
    value = raw.get(key)
    if value is None:
        return ()
    if isinstance(value, int) and not isinstance(value, bool):
        return (value,)
    if isinstance(value, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
        return tuple(value)
    raise ConfigError(f"{key} must be an integer or a list of integers")


@dataclass(frozen=True)
class LlamaConfig(ArchitectureConfig):
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    rope_scaling: Optional[Llama3Scaling] = None
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    architecture = "LlamaForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "LlamaConfig":
        hidden = _get(raw, "hidden_size", int)
        heads = _get(raw, "num_attention_heads", int)
        _positive("hidden_size", hidden)
        _positive("num_attention_heads", heads)
        if "head_dim" not in raw or raw["head_dim"] is None:
            if hidden % heads:
                raise ConfigError(
                    f"hidden_size {hidden} is no multiple of num_attention_heads {heads}; give head_dim")
            head_dim = hidden // heads
        else:
            head_dim = _get(raw, "head_dim", int)
        theta = raw.get("rope_theta")
        if theta is None and isinstance(raw.get("rope_parameters"), dict):
            theta = raw["rope_parameters"].get("rope_theta")
        if theta is None:
            raise ConfigError("config.json lacks the key 'rope_theta'")
        if isinstance(theta, bool) or not isinstance(theta, (int, float)):
            raise ConfigError(f"rope_theta must be a number, got {theta!r}")
        for key in ("attention_bias", "mlp_bias"):
            if _get(raw, key, bool, False):
                raise ConfigError(f"{key}=true is not supported by this LlamaForCausalLM implementation")
        bos = raw.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError("bos_token_id must be an integer")
        dtype = raw.get("torch_dtype", raw.get("dtype", "bfloat16"))
        cfg = cls(
            num_hidden_layers=_get(raw, "num_hidden_layers", int),
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=_get(raw, "num_key_value_heads", int, heads),
            head_dim=head_dim,
            intermediate_size=_get(raw, "intermediate_size", int),
            vocab_size=_get(raw, "vocab_size", int),
            rope_theta=float(theta),
            rms_norm_eps=_get(raw, "rms_norm_eps", float),
            max_position_embeddings=_get(raw, "max_position_embeddings", int),
            tie_word_embeddings=_get(raw, "tie_word_embeddings", bool, False),
            rope_scaling=_read_scaling(raw),
            eos_token_id=_read_token_ids(raw, "eos_token_id"),
            bos_token_id=bos,
            torch_dtype=str(dtype),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                     "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings",
                     "rope_theta", "rms_norm_eps"):
            _positive(name, getattr(self, name))
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is no multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        for tok in self.eos_token_id:
            if not 0 <= tok < self.vocab_size:
                raise ConfigError(f"eos_token_id {tok} lies outside the vocabulary of {self.vocab_size}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
            "rope_scaling": None,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            out["rope_scaling"] = {
                "rope_type": "llama3",
                "factor": s.factor,
                "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position,
            }
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) > 1 else self.eos_token_id[0]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out

    # ------------------------------------------------------------------ meaning
    def stop_token_ids(self) -> tuple:
        return tuple(self.eos_token_id)

    def max_positions(self) -> int:
        return self.max_position_embeddings

    def layout(self) -> ModelLayout:
        """Every layer alike: RMSNorm, grouped-query attention with rotary
        positions over all earlier keys, RMSNorm, SwiGLU; then the final norm
        and the head (inference/TransformerBlock.java:73-149,
        inference/InferenceEngine.java:225-262)."""
        position = PositionSpec(
            kind="rope", head_dim=self.head_dim, rotary_dim=self.head_dim,
            theta=self.rope_theta, scaling=self.rope_scaling, pairing="split_half")
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            layers.append(BlockSpec(
                mixer_norm=NormSpec(self.hidden_size, self.rms_norm_eps, p + "input_layernorm.weight"),
                mixer=AttentionSpec(
                    hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                    scale=1.0 / math.sqrt(self.head_dim), position=position,
                    q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight",
                    v=p + "self_attn.v_proj.weight", o=p + "self_attn.o_proj.weight"),
                ffn_norm=NormSpec(self.hidden_size, self.rms_norm_eps, p + "post_attention_layernorm.weight"),
                ffn=SwiGLUSpec(
                    hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                    gate=p + "mlp.gate_proj.weight", up=p + "mlp.up_proj.weight",
                    down=p + "mlp.down_proj.weight"),
            ))
        embed_name = "model.embed_tokens.weight"
        return ModelLayout(
            embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, embed_name),
            layers=tuple(layers),
            head=HeadSpec(
                self.vocab_size, self.hidden_size,
                norm=NormSpec(self.hidden_size, self.rms_norm_eps, "model.norm.weight"),
                weight=embed_name if self.tie_word_embeddings else "lm_head.weight"),
        )

    def describe(self) -> str:
        """One line per quantity, as the reference prints its configuration on
        load (model/ModelConfig.java:504-527)."""
        rows = [(k, v) for k, v in self.to_dict().items() if k not in ("architectures",)]
        width = max(len(k) for k, _ in rows)
        return "\n".join([f"architecture: {self.architecture}"] + [f"  {k.ljust(width)} = {v}" for k, v in rows])


register_architecture(LlamaConfig.architecture, LlamaConfig)
