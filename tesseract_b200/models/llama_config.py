"""Typed configuration of ``LlamaForCausalLM``, read from ``config.json``.

The reader mirrors the keys that the reference's Llama module reads
(src/model/llama_3_2.rs:72-94) and its validation (src/model/llama_3_2.rs:108-174),
relaxed where the reference ties itself to one checkpoint: ``rope_scaling`` may
be absent or null, ``eos_token_id`` may be one integer, ``head_dim`` defaults to
``hidden_size / num_attention_heads`` and need not multiply back to
``hidden_size``, and ``torch_dtype`` may be ``float32``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.reading import ConfigError, require as _require


@dataclass(frozen=True)
class RopeScaling:
    """Llama-3 frequency scaling (src/model/llama_3_2.rs:63-70)."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RopeScaling":
        rope_type = data.get("rope_type", data.get("type"))
        if rope_type is None:
            raise ConfigError("rope_scaling: missing 'rope_type'")
        if rope_type != "llama3":
            raise ConfigError(f"rope_scaling: unsupported rope_type '{rope_type}' (only 'llama3')")
        out = cls(
            rope_type=rope_type,
            factor=float(_require(data, "factor", (int, float), "rope_scaling")),
            low_freq_factor=float(_require(data, "low_freq_factor", (int, float), "rope_scaling")),
            high_freq_factor=float(_require(data, "high_freq_factor", (int, float), "rope_scaling")),
            original_max_position_embeddings=int(
                _require(data, "original_max_position_embeddings", int, "rope_scaling")
            ),
        )
        if (
            out.factor <= 0
            or out.low_freq_factor <= 0
            or out.high_freq_factor <= 0
            or out.original_max_position_embeddings <= 0
        ):
            raise ConfigError("rope_scaling: factors and original_max_position_embeddings must be positive")
        if out.high_freq_factor == out.low_freq_factor:
            raise ConfigError("rope_scaling: high_freq_factor must differ from low_freq_factor")
        return out

    def to_dict(self) -> dict:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass(frozen=True)
class LlamaConfig:
    """Every constant of a ``LlamaForCausalLM`` checkpoint."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    bos_token_id: int
    eos_token_id: Tuple[int, ...]
    torch_dtype: str = "bfloat16"
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    model_type: str = "llama"
    architectures: Tuple[str, ...] = ("LlamaForCausalLM",)

    ARCHITECTURE = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "LlamaConfig":
        architectures = tuple(data.get("architectures") or ())
        hidden_size = _require(data, "hidden_size", int)
        heads = _require(data, "num_attention_heads", int)
        if heads <= 0:
            raise ConfigError("num_attention_heads must be positive")
        head_dim = data.get("head_dim")
        if head_dim is None:
            if hidden_size % heads:
                raise ConfigError("head_dim is absent and hidden_size is not divisible by num_attention_heads")
            head_dim = hidden_size // heads
        rope_parameters = data.get("rope_parameters") or {}
        rope_theta = data.get("rope_theta", rope_parameters.get("rope_theta"))
        if rope_theta is None:
            raise ConfigError("config.json: missing required key 'rope_theta'")
        scaling = data.get("rope_scaling")
        if scaling is None and rope_parameters.get("rope_type") not in (None, "default"):
            scaling = rope_parameters
        if scaling is not None and scaling.get("rope_type", scaling.get("type")) == "default":
            scaling = None
        eos = data.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(e) for e in eos)
        cfg = cls(
            hidden_size=hidden_size,
            intermediate_size=_require(data, "intermediate_size", int),
            num_hidden_layers=_require(data, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=int(data.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            vocab_size=_require(data, "vocab_size", int),
            max_position_embeddings=_require(data, "max_position_embeddings", int),
            rms_norm_eps=float(_require(data, "rms_norm_eps", (int, float))),
            rope_theta=float(rope_theta),
            rope_scaling=RopeScaling.from_dict(scaling) if scaling is not None else None,
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            bos_token_id=int(data.get("bos_token_id") if data.get("bos_token_id") is not None else 0),
            eos_token_id=eos_ids,
            torch_dtype=str(data.get("torch_dtype") or data.get("dtype") or "bfloat16"),
            hidden_act=str(data.get("hidden_act", "silu")),
            attention_bias=bool(data.get("attention_bias", False)),
            mlp_bias=bool(data.get("mlp_bias", False)),
            model_type=str(data.get("model_type", "llama")),
            architectures=architectures or (cls.ARCHITECTURE,),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        def bad(message: str):
            raise ConfigError(message)

        if self.ARCHITECTURE not in self.architectures:
            bad(f"Llama requires architectures to contain {self.ARCHITECTURE}, got {list(self.architectures)}")
        if self.model_type != "llama":
            bad(f"Llama requires model_type 'llama', got '{self.model_type}'")
        if self.torch_dtype not in ("bfloat16", "float32"):
            bad(f"torch_dtype must be bfloat16 or float32, got '{self.torch_dtype}'")
        if self.hidden_act != "silu":
            bad("Llama requires the SiLU gated feed-forward (hidden_act='silu')")
        if self.attention_bias or self.mlp_bias:
            bad("Llama uses no attention or feed-forward bias tensors")
        for name in ("num_hidden_layers", "hidden_size", "intermediate_size", "vocab_size", "head_dim",
                     "max_position_embeddings"):
            if getattr(self, name) <= 0:
                bad(f"{name} must be positive")
        if self.num_key_value_heads <= 0 or self.num_attention_heads % self.num_key_value_heads:
            bad("num_attention_heads must be a positive multiple of num_key_value_heads")
        if self.head_dim % 2:
            bad("head_dim must be even for rotate-half position encoding")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            bad("rms_norm_eps must be finite and positive")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            bad("rope_theta must be finite and positive")
        if self.rope_scaling is not None:
            if self.max_position_embeddings < self.rope_scaling.original_max_position_embeddings:
                bad("max_position_embeddings is smaller than the original rope context")
        if not 0 <= self.bos_token_id < self.vocab_size:
            bad("bos_token_id must lie inside the vocabulary")
        if any(not 0 <= t < self.vocab_size for t in self.eos_token_id):
            bad("eos_token_id must lie inside the vocabulary")

    def to_dict(self) -> dict:
        return {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "torch_dtype": self.torch_dtype,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": list(self.eos_token_id),
        }
