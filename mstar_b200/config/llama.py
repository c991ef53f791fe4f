"""Typed configuration of the dense Llama decoder ("LlamaForCausalLM").

Field names are the config.json keys.  The reference keeps the same names in
a dataclass with literal Llama-3.2-3B defaults and never opens config.json
(mstar/model/orpheus/config.py:4-53, mstar/model/orpheus/orpheus_model.py:71);
here nothing has a size default: what config.json does not give is an error.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Mapping, Optional

from .base import ConfigError, ModelConfig, optional, require
from .layout import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelLayout, NormSpec,
                     PositionSpec, RopeScalingSpec, RunEntry)

_ROPE_SCALING_KEYS = ("factor", "low_freq_factor", "high_freq_factor",
                      "original_max_position_embeddings")


@dataclass
class LlamaConfig(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: Optional[dict] = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Any = None
    pad_token_id: Optional[int] = None
    architectures: list = field(default_factory=lambda: ["LlamaForCausalLM"])

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        missing: list[str] = []
        hidden = require(raw, "hidden_size", int, missing)
        heads = require(raw, "num_attention_heads", int, missing)
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=require(raw, "intermediate_size", int, missing),
            num_hidden_layers=require(raw, "num_hidden_layers", int, missing),
            num_attention_heads=heads,
            num_key_value_heads=optional(raw, "num_key_value_heads", int, heads),
            head_dim=optional(raw, "head_dim", int, hidden // heads if heads else 0),
            vocab_size=require(raw, "vocab_size", int, missing),
            rms_norm_eps=require(raw, "rms_norm_eps", float, missing),
            rope_theta=require(raw, "rope_theta", float, missing),
            max_position_embeddings=require(raw, "max_position_embeddings", int, missing),
            rope_scaling=raw.get("rope_scaling"),
            tie_word_embeddings=optional(raw, "tie_word_embeddings", bool, False),
            hidden_act=optional(raw, "hidden_act", str, "silu"),
            attention_bias=optional(raw, "attention_bias", bool, False),
            mlp_bias=optional(raw, "mlp_bias", bool, False),
            torch_dtype=optional(raw, "torch_dtype", str, None)
            or optional(raw, "dtype", str, "bfloat16"),
            bos_token_id=optional(raw, "bos_token_id", int, None),
            eos_token_id=raw.get("eos_token_id"),
            pad_token_id=optional(raw, "pad_token_id", int, None),
            architectures=list(raw.get("architectures") or ["LlamaForCausalLM"]),
        )
        if missing:
            raise ConfigError("config.json lacks the keys " + ", ".join(sorted(missing))
                              + " that LlamaForCausalLM needs")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        problems: list[str] = []
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
                    "max_position_embeddings"):
            if getattr(self, key) <= 0:
                problems.append(f"{key} must be positive, got {getattr(self, key)}")
        if not problems:
            if self.num_attention_heads % self.num_key_value_heads:
                problems.append(
                    f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                    f"num_key_value_heads ({self.num_key_value_heads})")
            if self.head_dim % 2:
                problems.append(f"head_dim ({self.head_dim}) must be even for rotary pairs")
        if self.rms_norm_eps <= 0:
            problems.append(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_theta <= 0:
            problems.append(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            problems.append(f"hidden_act {self.hidden_act!r} is not supported (silu only)")
        if self.attention_bias:
            problems.append("attention_bias=true is not supported")
        if self.mlp_bias:
            problems.append("mlp_bias=true is not supported")
        if self.rope_scaling is not None:
            if not isinstance(self.rope_scaling, dict):
                problems.append("rope_scaling must be an object or null")
            else:
                kind = self.rope_scaling.get("rope_type", self.rope_scaling.get("type"))
                if kind in (None, "default"):
                    pass
                elif kind != "llama3":
                    problems.append(f"rope_scaling.rope_type {kind!r} is not supported "
                                    "(known: llama3, default)")
                else:
                    absent = [k for k in _ROPE_SCALING_KEYS if k not in self.rope_scaling]
                    if absent:
                        problems.append("rope_scaling lacks " + ", ".join(absent))
        if problems:
            raise ConfigError("unusable Llama configuration: " + "; ".join(problems))

    def to_dict(self) -> dict:
        out = asdict(self)
        out["architectures"] = list(self.architectures)
        return out

    def _scaling_spec(self) -> Optional[RopeScalingSpec]:
        rs = self.rope_scaling
        if not rs or rs.get("rope_type", rs.get("type")) in (None, "default"):
            return None
        return RopeScalingSpec(
            rope_type="llama3",
            factor=float(rs["factor"]),
            low_freq_factor=float(rs["low_freq_factor"]),
            high_freq_factor=float(rs["high_freq_factor"]),
            original_max_position_embeddings=int(rs["original_max_position_embeddings"]),
        )

    def layout(self) -> ModelLayout:
        """Every layer is the same pre-norm block (mstar/model/orpheus/components/
        language_model.py:30-52): GQA attention with llama3-scaled rotary positions,
        SwiGLU feed-forward, two RMSNorms; layers run once each, in order, each with
        a cache of its own."""
        position = PositionSpec(kind="rope", head_dim=self.head_dim, rotary_dim=self.head_dim,
                                theta=self.rope_theta, scaling=self._scaling_spec(),
                                interleaved=False)
        mixer = AttentionSpec(hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                              num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                              position=position, window=None, scale=None)
        ffn = GatedMLPSpec(hidden_size=self.hidden_size,
                           intermediate_size=self.intermediate_size,
                           activation=self.hidden_act)
        norm = NormSpec(kind="rmsnorm", size=self.hidden_size, eps=self.rms_norm_eps)
        block = BlockSpec(kind="prenorm", mixer=mixer, ffn=ffn, norm1=norm, norm2=norm)
        blocks = [block for _ in range(self.num_hidden_layers)]
        order = [RunEntry(block=i, cache=i) for i in range(self.num_hidden_layers)]
        layout = ModelLayout(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                             blocks=blocks, order=order, final_norm=norm,
                             tie_word_embeddings=self.tie_word_embeddings,
                             max_positions=self.max_position_embeddings)
        layout.validate()
        return layout

    def stop_token_ids(self) -> tuple[int, ...]:
        eos = self.eos_token_id
        if eos is None:
            return ()
        if isinstance(eos, (list, tuple)):
            return tuple(int(t) for t in eos)
        return (int(eos),)

    def max_positions(self) -> int:
        return self.max_position_embeddings
