"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference obtains its configuration object from ``transformers.LlamaConfig``
(tokasaurus/model/llama.py:13,605,784) and reads these attributes from it:
``hidden_size``, ``num_attention_heads``, ``num_key_value_heads``
(llama.py:104-127,158-159), ``num_hidden_layers`` (llama.py:538-546),
``intermediate_size`` (llama.py:299-316), ``vocab_size`` (llama.py:437-439,511-513),
``rms_norm_eps`` (llama.py:47), ``max_position_embeddings`` and the rope keys
(llama.py:559-570), ``tie_word_embeddings`` (llama.py:842-845).  Only those keys
are read here; every size in the engine comes from this object.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can run."""


@dataclass(frozen=True)
class RopeScaling:
    """The ``rope_scaling`` dictionary of config.json.

    ``rope_type`` is ``"default"`` (plain rotary encoding) or ``"llama3"`` (frequency
    dependent stretching of long wavelengths).
    """

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @staticmethod
    def from_dict(d: dict[str, Any] | None) -> "RopeScaling | None":
        if d is None:
            return None
        rope_type = d.get("rope_type", d.get("type", "default"))
        if rope_type not in ("default", "llama3"):
            raise ConfigError(
                f"rope_scaling.rope_type={rope_type!r} is not supported (known: 'default', 'llama3')"
            )
        if rope_type == "default":
            return RopeScaling()
        missing = [
            k
            for k in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
            if k not in d
        ]
        if missing:
            raise ConfigError(f"rope_scaling of type 'llama3' lacks keys {missing}")
        rs = RopeScaling(
            rope_type="llama3",
            factor=float(d["factor"]),
            low_freq_factor=float(d["low_freq_factor"]),
            high_freq_factor=float(d["high_freq_factor"]),
            original_max_position_embeddings=int(d["original_max_position_embeddings"]),
        )
        if rs.high_freq_factor == rs.low_freq_factor:
            raise ConfigError("rope_scaling: high_freq_factor must differ from low_freq_factor")
        if rs.factor <= 0:
            raise ConfigError("rope_scaling: factor must be positive")
        return rs

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


@dataclass(frozen=True)
class LlamaConfig:
    """Configuration of the dense Llama decoder (config.json key names)."""

    hidden_size: int
    num_attention_heads: int
    num_hidden_layers: int
    intermediate_size: int
    vocab_size: int
    num_key_value_heads: int | None = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 2048
    eos_token_id: tuple[int, ...] = ()
    architectures: tuple[str, ...] = ("LlamaForCausalLM",)
    model_type: str = "llama"
    extra: dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    REQUIRED = ("hidden_size", "num_attention_heads", "num_hidden_layers", "intermediate_size", "vocab_size")

    def __post_init__(self) -> None:
        if self.num_key_value_heads is None:
            object.__setattr__(self, "num_key_value_heads", self.num_attention_heads)
        for name in self.REQUIRED + ("num_key_value_heads", "max_position_embeddings"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        if self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"hidden_size={self.hidden_size} is not a multiple of num_attention_heads={self.num_attention_heads}"
            )
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary encoding")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            raise ConfigError(f"rms_norm_eps must be positive and finite, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0 and math.isfinite(self.rope_theta)):
            raise ConfigError(f"rope_theta must be positive and finite, got {self.rope_theta!r}")

    @property
    def head_dim(self) -> int:
        # hidden_size // num_attention_heads, as tokasaurus/model/llama.py:158-159 computes it;
        # a separate "head_dim" key is not part of this architecture.
        return self.hidden_size // self.num_attention_heads

    @property
    def num_query_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "LlamaConfig":
        missing = [k for k in LlamaConfig.REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks required keys {missing}")
        known = {
            "hidden_size", "num_attention_heads", "num_hidden_layers", "intermediate_size", "vocab_size",
            "num_key_value_heads", "rms_norm_eps", "rope_theta", "rope_scaling", "tie_word_embeddings",
            "max_position_embeddings", "eos_token_id", "architectures", "model_type", "head_dim",
        }
        if d.get("head_dim") is not None:
            want = int(d["hidden_size"]) // int(d["num_attention_heads"])
            if int(d["head_dim"]) != want:
                raise ConfigError(
                    f"head_dim={d['head_dim']} differs from hidden_size // num_attention_heads = {want}; "
                    "this architecture derives the head size from those two keys"
                )
        for flag in ("attention_bias", "mlp_bias"):
            if d.get(flag):
                raise ConfigError(f"{flag}=true is not part of this architecture (projections have no bias)")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act={d['hidden_act']!r} is not supported; the feed-forward uses 'silu'")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_t: tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_t = (eos,)
        else:
            eos_t = tuple(int(e) for e in eos)
        kv = d.get("num_key_value_heads")
        return LlamaConfig(
            hidden_size=d["hidden_size"],
            num_attention_heads=d["num_attention_heads"],
            num_hidden_layers=d["num_hidden_layers"],
            intermediate_size=d["intermediate_size"],
            vocab_size=d["vocab_size"],
            num_key_value_heads=kv if kv is not None else None,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            eos_token_id=eos_t,
            architectures=tuple(d.get("architectures") or ("LlamaForCausalLM",)),
            model_type=str(d.get("model_type", "llama")),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu",
        }
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) > 1 else self.eos_token_id[0]
        return out


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in model folder {str(model_dir)!r}")
    with open(path) as f:
        d = json.load(f)
    if not isinstance(d, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return d


def read_eos_token_ids(model_dir: str | Path, config_dict: dict[str, Any]) -> tuple[int, ...]:
    """EOS ids: generation_config.json's ``eos_token_id`` (int or list) as in
    tokasaurus/utils.py:447-457, else config.json's, else none."""
    gen = Path(model_dir) / "generation_config.json"
    eos = None
    if gen.is_file():
        with open(gen) as f:
            eos = json.load(f).get("eos_token_id")
    if eos is None:
        eos = config_dict.get("eos_token_id")
    if eos is None:
        return ()
    if isinstance(eos, int):
        return (eos,)
    return tuple(int(e) for e in eos)
