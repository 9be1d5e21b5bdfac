"""The dense Llama decoder as a ``ModelSpec``: which parts, with which constants, under which
tensor names.  Structure and names are those of umarhassan-cloud/kvforge's ``Transformer``
(src/tokenvault/model.py:146-163; checkpoint names carry the ``model.`` prefix that
src/tokenvault/model_loader.py:104 strips)."""

from __future__ import annotations

from ..config.model_config import ModelConfig
from ..parts.base import PartSpec
from ..parts.model import LayerCall, LayerSpec, ModelSpec


def llama_spec(cfg: ModelConfig) -> ModelSpec:
    position = PartSpec(
        "rotary",
        {
            "head_dim": cfg.head_dim,
            "theta": cfg.rope_theta,
            "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
        },
    )
    norm = PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    mixer = PartSpec(
        "paged_attention",
        {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_heads,
            "num_kv_heads": cfg.num_kv_heads,
            "head_dim": cfg.head_dim,
            "position": position,
            "window": None,
        },
    )
    ffn = PartSpec(
        "gated_mlp",
        {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size, "activation": cfg.hidden_act},
    )
    layers = [
        LayerSpec(
            block=PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn}),
            prefix=f"model.layers.{i}.",
        )
        for i in range(cfg.num_layers)
    ]
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=layers,
        final_norm=norm,
        execution=[LayerCall(i) for i in range(cfg.num_layers)],
        tie_word_embeddings=cfg.tie_word_embeddings,
        max_position_embeddings=cfg.max_position_embeddings,
        eos_token_id=cfg.eos_token_id,
        bos_token_id=cfg.bos_token_id,
    )
