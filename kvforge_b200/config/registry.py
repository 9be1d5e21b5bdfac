"""The one registry from an architecture's name (``config.json``'s ``architectures[0]``) to
how its configuration is read and its model is described, and the named presets.

umarhassan-cloud/kvforge has a single model class and a ``PRESETS`` table
(src/tokenvault/model_loader.py:17-39); the presets here are the shapes this engine is
measured and tested on, with the llama3 frequency scaling those checkpoints carry.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .model_config import ConfigError, ModelConfig, RopeScaling


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict[str, Any]], Any]  # config.json dict -> typed config
    build_spec: Callable[[Any], Any]  # typed config -> parts.model.ModelSpec


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable, build_spec: Callable) -> None:
    if name in ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def unregister_architecture(name: str) -> None:
    ARCHITECTURES.pop(name, None)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered (known: {sorted(ARCHITECTURES)})")
    return ARCHITECTURES[name]


def architecture_of(config_json: dict[str, Any]) -> Architecture:
    archs = config_json.get("architectures")
    if not archs:
        raise ConfigError("config.json names no architecture (key 'architectures')")
    return get_architecture(archs[0])


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from ..models.llama import llama_spec

    if "LlamaForCausalLM" not in ARCHITECTURES:
        register_architecture("LlamaForCausalLM", ModelConfig.from_hf_dict, llama_spec)


_LLAMA3_32 = RopeScaling(factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
_LLAMA3_8 = RopeScaling(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)

PRESETS: dict[str, ModelConfig] = {
    "tiny-a": ModelConfig(
        vocab_size=256, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
        intermediate_size=192, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True,
        max_position_embeddings=128,
    ),
    "tiny-b": ModelConfig(
        vocab_size=320, hidden_size=96, num_layers=3, num_heads=3, num_kv_heads=1, head_dim=32,
        intermediate_size=256, rms_norm_eps=1e-6, rope_theta=500000.0,
        rope_scaling=RopeScaling(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64),
        tie_word_embeddings=False, max_position_embeddings=256,
    ),
    "llama-3.2-1b": ModelConfig(
        vocab_size=128256, hidden_size=2048, num_layers=16, num_heads=32, num_kv_heads=8, head_dim=64,
        intermediate_size=8192, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=_LLAMA3_32,
        tie_word_embeddings=True, max_position_embeddings=131072, bos_token_id=128000, eos_token_id=128001,
    ),
    "llama-3.2-3b": ModelConfig(
        vocab_size=128256, hidden_size=3072, num_layers=28, num_heads=24, num_kv_heads=8, head_dim=128,
        intermediate_size=8192, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=_LLAMA3_32,
        tie_word_embeddings=True, max_position_embeddings=131072, bos_token_id=128000, eos_token_id=128001,
    ),
    "llama-3.1-8b": ModelConfig(
        vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8, head_dim=128,
        intermediate_size=14336, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=_LLAMA3_8,
        tie_word_embeddings=False, max_position_embeddings=131072, bos_token_id=128000, eos_token_id=128001,
    ),
}  # fmt: skip
# kvforge's own preset name for the 1B shape (src/tokenvault/model_loader.py:28-33)
PRESETS["llama-1b"] = PRESETS["llama-3.2-1b"]
PRESETS["llama-8b"] = PRESETS["llama-3.1-8b"]
