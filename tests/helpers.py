"""Shared by the tests: the two tiny configurations, model folders in temporary
directories, and error measures."""

from __future__ import annotations

import random
from pathlib import Path

import torch

from kvforge_b200 import PRESETS, ModelConfig, RopeScaling
from kvforge_b200.models.folder import write_random_model

# tiny-a and tiny-b differ in every size and option: layers, width, heads, groups, head size,
# intermediate size, vocabulary, theta, scaling, eps, tying, block size.
TINY = {
    "tiny-a": dict(cfg=PRESETS["tiny-a"], block_size=16),
    "tiny-b": dict(cfg=PRESETS["tiny-b"], block_size=8),
    # head_dim * heads != hidden, vocabulary and width no powers of two
    "tiny-c": dict(
        cfg=ModelConfig(
            vocab_size=203, hidden_size=80, num_layers=2, num_heads=6, num_kv_heads=3, head_dim=48,
            intermediate_size=112, rms_norm_eps=3e-6, rope_theta=25000.0,
            rope_scaling=RopeScaling(factor=4.0, low_freq_factor=1.0, high_freq_factor=2.0, original_max_position_embeddings=32),
            tie_word_embeddings=False, max_position_embeddings=512,
        ),
        block_size=4,
    ),
    # head size 64 with four heads per kv head and pages of 16: in bfloat16 the tcgen05 kernel takes
    # its prompts and mixed batches, the TMA kernel its decode steps
    "tiny-d": dict(
        cfg=ModelConfig(
            vocab_size=211, hidden_size=96, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=64,
            intermediate_size=160, rms_norm_eps=2e-5, rope_theta=10000.0, tie_word_embeddings=True,
            max_position_embeddings=512,
        ),
        block_size=16,
    ),
    # head size 128 with two heads per kv head and pages of 32 (the sizes of the larger shapes in small):
    # the same two kernels with tiles of two halves and boxes of 32 keys
    "tiny-e": dict(
        cfg=ModelConfig(
            vocab_size=157, hidden_size=128, num_layers=3, num_heads=4, num_kv_heads=2, head_dim=128,
            intermediate_size=96, rms_norm_eps=1e-5, rope_theta=50000.0, tie_word_embeddings=False,
            max_position_embeddings=512,
        ),
        block_size=32,
    ),
}  # fmt: skip


def make_model_dir(tmp: Path, name: str, seed: int = 11, store_dtype=torch.float32, init_std: float = 0.1) -> Path:
    """A model folder with weights large enough that attention and norms matter."""
    d = Path(tmp) / f"{name}-{seed}"
    if not d.exists():
        write_random_model(d, TINY[name]["cfg"], seed=seed, store_dtype=store_dtype, init_std=init_std, norm_std=0.1)
    return d


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max())


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """Largest difference relative to the largest reference magnitude."""
    return max_abs(a, b) / max(float(b.double().abs().max()), 1e-30)
