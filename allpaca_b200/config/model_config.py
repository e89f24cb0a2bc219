"""Typed model configuration for the dense Llama decoder.

Every size and constant of the model comes from the keys of the
architecture's own ``config.json``; nothing is hard-coded elsewhere.

Reference parity: the key set and the defaults follow the reference's serde
view of ``config.json`` (crates/allpaca-safetensors/src/sidecar.rs:136-229):
``vocab_size`` 32, ``hidden_size`` 32, ``num_hidden_layers`` 1,
``num_attention_heads`` 4, ``num_key_value_heads`` -> heads,
``intermediate_size`` -> 4*hidden (crates/allpaca-core/src/model.rs:7922),
``head_dim`` -> hidden/heads (model.rs:366-372), ``rms_norm_eps`` 1e-5,
``rope_theta`` 10000.  ``hidden_act`` must be a SiLU spelling
(sidecar.rs:239-247).  ``rope_scaling`` (llama3 frequency scaling) and
``max_position_embeddings`` are additions of this engine: the reference has
no field for them (model.rs:181-274).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine runs."""


_SILU_NAMES = ("silu", "swish", "silu_and_mul")


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of rotary embeddings (``rope_scaling`` in config.json)."""

    rope_type: str = "llama3"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RopeScaling":
        rope_type = d.get("rope_type", d.get("type"))
        if rope_type != "llama3":
            raise ConfigError(
                f"rope_scaling.rope_type {rope_type!r} is not supported (known: 'llama3')")
        try:
            out = cls(
                rope_type="llama3",
                factor=float(d["factor"]),
                low_freq_factor=float(d.get("low_freq_factor", 1.0)),
                high_freq_factor=float(d.get("high_freq_factor", 4.0)),
                original_max_position_embeddings=int(
                    d["original_max_position_embeddings"]),
            )
        except KeyError as e:
            raise ConfigError(f"rope_scaling lacks key {e.args[0]!r}") from None
        if out.factor <= 0:
            raise ConfigError("rope_scaling.factor must be positive")
        if out.high_freq_factor <= out.low_freq_factor:
            raise ConfigError(
                "rope_scaling.high_freq_factor must exceed low_freq_factor")
        if out.original_max_position_embeddings <= 0:
            raise ConfigError(
                "rope_scaling.original_max_position_embeddings must be positive")
        return out

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class LlamaConfig:
    """The hyper-parameters of one dense Llama decoder, as config.json gives them."""

    vocab_size: int = 32
    hidden_size: int = 32
    num_hidden_layers: int = 1
    num_attention_heads: int = 4
    num_key_value_heads: int = 4
    head_dim: int = 8
    intermediate_size: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 2048
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    architectures: tuple = ("LlamaForCausalLM",)
    model_type: str = "llama"

    # ---- derived sizes -------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def architecture(self) -> str:
        return self.architectures[0] if self.architectures else self.model_type

    # ---- construction --------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        def integer(key: str, default: Optional[int]) -> Optional[int]:
            v = d.get(key, default)
            if v is None:
                return None
            if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
                raise ConfigError(f"{key} must be an integer, got {v!r}")
            return int(v)

        hidden = integer("hidden_size", 32)
        heads = integer("num_attention_heads", 4)
        kv_heads = integer("num_key_value_heads", None)
        if kv_heads is None:
            kv_heads = heads
        head_dim = integer("head_dim", None)
        if heads is None or heads <= 0:
            raise ConfigError("num_attention_heads must be positive")
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"hidden_size {hidden} is not divisible by num_attention_heads "
                    f"{heads} and head_dim is not given")
            head_dim = hidden // heads
        inter = integer("intermediate_size", None)
        if inter is None:
            inter = 4 * hidden
        act = d.get("hidden_act")
        if act is None:
            act = "silu"
        if str(act).lower() not in _SILU_NAMES:
            raise ConfigError(
                f"hidden_act {act!r} is not supported (known: {', '.join(_SILU_NAMES)})")
        for moe_key in ("num_local_experts", "n_routed_experts", "num_experts",
                        "num_experts_per_tok"):
            if d.get(moe_key):
                raise ConfigError(
                    f"{moe_key} is set: mixture-of-experts checkpoints are not a dense Llama")
        for bias_key in ("attention_bias", "mlp_bias"):
            if d.get(bias_key):
                raise ConfigError(
                    f"{bias_key} is set: projections with biases are not part of this architecture "
                    f"(the reference's Llama path has none)")
        scaling = d.get("rope_scaling")
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type"))
            scaling = None if kind in (None, "default") else RopeScaling.from_dict(scaling)
        archs = d.get("architectures") or ()
        if isinstance(archs, str):
            archs = (archs,)
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"
        cfg = cls(
            vocab_size=integer("vocab_size", 32),
            hidden_size=hidden,
            num_hidden_layers=integer("num_hidden_layers", 1),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=inter,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=scaling,
            tie_word_embeddings=bool(d.get("tie_word_embeddings") or False),
            max_position_embeddings=integer("max_position_embeddings", 2048),
            hidden_act="silu",
            torch_dtype=str(dtype).replace("torch.", ""),
            architectures=tuple(archs),
            model_type=str(d.get("model_type") or "llama"),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:
        pos = {
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
        }
        for k, v in pos.items():
            if v <= 0:
                raise ConfigError(f"{k} must be positive, got {v}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            # crates/allpaca-cpu/src/kernels.rs:306-310
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            # crates/allpaca-cpu/src/kernels.rs:511
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        if not (self.rope_theta > 0):
            raise ConfigError("rope_theta must be positive")

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["rope_scaling"] = self.rope_scaling.to_dict() if self.rope_scaling else None
        return d


def read_config_json(path: str) -> dict:
    """Read ``config.json`` from a file or a model folder."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return d
