"""Typed configuration of the Llama dense decoder, read from its own config.json keys.

The reference reads the same keys in picolm/safetensors.c:44-136
(`hidden_size intermediate_size num_attention_heads num_key_value_heads
num_hidden_layers vocab_size head_dim rms_norm_eps rope_theta`) and the GGUF
twins in picolm/model_gguf.c:755-903.  Defaults of absent keys follow the
reference: `head_dim = hidden_size / num_attention_heads`
(picolm/safetensors.c:75-76), `rms_norm_eps = 1e-6` (picolm/safetensors.c:77-78),
`rope_theta = 10000` (picolm/safetensors.c:101-102), `bos/eos = 1/2`
(picolm/safetensors.c:327-330).  The reference has no `rope_scaling`; the
`llama3` rule is read here because Llama-3 checkpoints carry it.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that this library cannot run, with the key named."""


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of a Llama-3 checkpoint (rope_type "llama3")."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Optional[Mapping[str, Any]]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(
                f"rope_scaling.rope_type={kind!r} is not supported (supported: 'llama3', 'default' or absent)")
        try:
            out = RopeScaling(
                rope_type="llama3",
                factor=float(d["factor"]),
                low_freq_factor=float(d["low_freq_factor"]),
                high_freq_factor=float(d["high_freq_factor"]),
                original_max_position_embeddings=int(d["original_max_position_embeddings"]),
            )
        except KeyError as e:
            raise ConfigError(f"rope_scaling of type 'llama3' lacks the key {e.args[0]!r}") from None
        if out.factor <= 0 or out.original_max_position_embeddings <= 0:
            raise ConfigError("rope_scaling.factor and original_max_position_embeddings must be positive")
        if out.high_freq_factor <= out.low_freq_factor:
            raise ConfigError("rope_scaling.high_freq_factor must exceed low_freq_factor")
        return out

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)


def _as_id_tuple(v: Any, default: Tuple[int, ...]) -> Tuple[int, ...]:
    if v is None:
        return default
    if isinstance(v, (list, tuple)):
        return tuple(int(x) for x in v)
    return (int(v),)


@dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of one Llama checkpoint.  Nothing here has a
    model-specific value in code: each field comes from config.json or from the
    reference's default for an absent key."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    bos_token_id: int = 1
    eos_token_id: Tuple[int, ...] = (2,)
    torch_dtype: str = "bfloat16"
    architecture: str = "LlamaForCausalLM"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)

    # ------------------------------------------------------------------ read
    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "LlamaConfig":
        # A multimodal wrapper keeps the decoder's keys under text_config
        # (picolm/safetensors.c:66-67).
        d = raw.get("text_config") if isinstance(raw.get("text_config"), dict) else raw

        def need(key: str) -> int:
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json lacks the key {key!r}")
            return int(d[key])

        hidden = need("hidden_size")
        heads = need("num_attention_heads")
        if heads <= 0:
            raise ConfigError("num_attention_heads must be positive")
        kv_heads = d.get("num_key_value_heads")
        head_dim = d.get("head_dim")
        eps = d.get("rms_norm_eps")
        theta = d.get("rope_theta")
        archs = raw.get("architectures") or ["LlamaForCausalLM"]
        known = {
            "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "rope_scaling",
            "max_position_embeddings", "tie_word_embeddings", "hidden_act", "attention_bias", "mlp_bias",
            "bos_token_id", "eos_token_id", "torch_dtype", "dtype", "architectures",
        }
        cfg = LlamaConfig(
            vocab_size=need("vocab_size"),
            hidden_size=hidden,
            intermediate_size=need("intermediate_size"),
            num_hidden_layers=need("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(kv_heads) if kv_heads else heads,
            head_dim=int(head_dim) if head_dim else hidden // heads,
            rms_norm_eps=float(eps) if eps else 1e-6,
            rope_theta=float(theta) if theta and float(theta) > 0 else 10000.0,
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            max_position_embeddings=int(d.get("max_position_embeddings") or 2048),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            attention_bias=bool(d.get("attention_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
            bos_token_id=int(d["bos_token_id"]) if d.get("bos_token_id") is not None else 1,
            eos_token_id=_as_id_tuple(d.get("eos_token_id"), (2,)),
            torch_dtype=str(d.get("torch_dtype") or d.get("dtype") or "bfloat16"),
            architecture=str(archs[0]),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @staticmethod
    def from_json(path: str) -> "LlamaConfig":
        with open(path, "r", encoding="utf-8") as f:
            return LlamaConfig.from_dict(json.load(f))

    # -------------------------------------------------------------- validate
    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        # The reference hard-codes SiLU and has no bias tensors
        # (picolm/model_core.c:2192-2193, picolm/model_core.c:1849-2220).
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act={self.hidden_act!r} is not supported (only 'silu')")
        if self.attention_bias:
            raise ConfigError("attention_bias=true is not supported")
        if self.mlp_bias:
            raise ConfigError("mlp_bias=true is not supported")

    # ----------------------------------------------------------------- write
    def to_dict(self) -> dict:
        eos: Any = list(self.eos_token_id)
        if len(eos) == 1:
            eos = eos[0]
        out = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": eos,
            "torch_dtype": self.torch_dtype,
        }
        return out
