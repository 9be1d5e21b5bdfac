"""Typed model configuration read from the architecture's own ``config.json`` keys.

Field names follow umarhassan-cloud/kvforge's ``ModelConfig`` (src/tokenvault/config.py:34-72);
the mapping from ``config.json`` keys follows ``config_from_hf``
(src/tokenvault/model_loader.py:64-86).  The Gemma-only fields of that class are left out:
this engine builds the Llama decoder only and rejects what it does not implement.  Added:
``rope_scaling`` (the llama3 frequency scaling that Llama 3.1/3.2 checkpoints need and
kvforge lacks).
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A ``config.json`` that this engine cannot run, with the reason."""


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of ``config.json`` with ``rope_type == "llama3"``."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int
    rope_type: str = "llama3"

    @classmethod
    def from_dict(cls, d: dict[str, Any] | None) -> RopeScaling | None:
        if not d:
            return None
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"rope_scaling.rope_type {kind!r} is not supported (only 'llama3' or none)")
        missing = [
            k
            for k in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
            if k not in d
        ]
        if missing:
            raise ConfigError(f"rope_scaling lacks {missing}")
        hi, lo = float(d["high_freq_factor"]), float(d["low_freq_factor"])
        if hi <= lo:
            raise ConfigError("rope_scaling needs high_freq_factor > low_freq_factor")
        return cls(
            factor=float(d["factor"]),
            low_freq_factor=lo,
            high_freq_factor=hi,
            original_max_position_embeddings=int(d["original_max_position_embeddings"]),
        )

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


@dataclass
class ModelConfig:
    """Hyper-parameters of a dense decoder.  No default stands for a size: every size must
    be given (by ``config.json`` or by the caller)."""

    vocab_size: int
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    intermediate_size: int
    rms_norm_eps: float
    head_dim: int | None = None
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    hidden_act: str = "silu"
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    architectures: list[str] = field(default_factory=lambda: ["LlamaForCausalLM"])

    def __post_init__(self) -> None:
        # src/tokenvault/config.py:56-62
        if self.head_dim is None:
            if self.hidden_size % self.num_heads != 0:
                raise ConfigError("hidden_size must be divisible by num_heads when head_dim is unset")
            self.head_dim = self.hidden_size // self.num_heads
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads != 0:
            raise ConfigError("num_heads must be a multiple of num_kv_heads (GQA)")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        for name in ("vocab_size", "hidden_size", "num_layers", "num_heads", "intermediate_size", "head_dim"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if isinstance(self.rope_scaling, dict):
            self.rope_scaling = RopeScaling.from_dict(self.rope_scaling)

    @property
    def architecture(self) -> str:
        return self.architectures[0]

    @property
    def num_params(self) -> int:
        """Parameter count without norms (src/tokenvault/config.py:64-72)."""
        h, d = self.hidden_size, self.head_dim
        attn = h * d * (self.num_heads * 2 + self.num_kv_heads * 2)
        mlp = 3 * h * self.intermediate_size
        emb = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return self.num_layers * (attn + mlp) + emb

    # ------------------------------------------------------------------ config.json
    @classmethod
    def from_hf_dict(cls, d: dict[str, Any]) -> ModelConfig:
        """``config.json`` keys -> fields (src/tokenvault/model_loader.py:64-86)."""
        required = [
            "vocab_size",
            "hidden_size",
            "num_hidden_layers",
            "num_attention_heads",
            "intermediate_size",
            "rms_norm_eps",
            "max_position_embeddings",
        ]
        missing = [k for k in required if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks {missing}")
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ConfigError("attention_bias / mlp_bias are not supported (bias-free projections only)")
        act = d.get("hidden_activation") or d.get("hidden_act", "silu")
        eos = d.get("eos_token_id")
        if isinstance(eos, list):  # model_loader.py:68
            eos = eos[0] if eos else None
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        return cls(
            vocab_size=int(d["vocab_size"]),
            hidden_size=int(d["hidden_size"]),
            num_layers=int(d["num_hidden_layers"]),
            num_heads=int(d["num_attention_heads"]),
            num_kv_heads=int(d.get("num_key_value_heads") or d["num_attention_heads"]),
            intermediate_size=int(d["intermediate_size"]),
            head_dim=d.get("head_dim"),
            max_position_embeddings=int(d["max_position_embeddings"]),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            rms_norm_eps=float(d["rms_norm_eps"]),
            hidden_act=act,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=eos,
            architectures=list(archs),
        )

    def to_hf_dict(self) -> dict[str, Any]:
        out = {
            "architectures": list(self.architectures),
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "rms_norm_eps": self.rms_norm_eps,
            "hidden_act": self.hidden_act,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_id,
        }
        return out


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} not found")
    return json.loads(path.read_text())
