"""Writes a model folder (``config.json`` + ``model.safetensors``) with random weights from a
configuration and a seed: the random-weights mode as files, so that this engine and any
other program read the very same bytes."""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.registry import get_architecture
from ..parts.model import DecoderModel
from ..weights.random_init import write_model_dir


def write_random_model(
    model_dir: str | Path,
    config,
    seed: int = 0,
    store_dtype: torch.dtype = torch.bfloat16,
    init_std: float = 0.02,
    norm_std: float = 0.0,
    device: torch.device | str = "cpu",
) -> Path:
    """``config`` is a typed model configuration (its ``architectures[0]`` picks the model)."""
    arch = get_architecture(config.architectures[0])
    spec = arch.build_spec(config)
    model = DecoderModel(spec)
    skip = (spec.lm_head_name,) if spec.tie_word_embeddings else ()
    return write_model_dir(
        model_dir, config.to_hf_dict(), model.expected_weights(), seed, store_dtype, init_std, norm_std, skip, device
    )
