"""Cache, scheduler and engine configuration.

Names and meanings follow umarhassan-cloud/kvforge's ``CacheConfig``, ``SchedulerConfig`` and
``EngineConfig`` (src/tokenvault/config.py:75-151).  Left out: prefix caching, priority
policy, speculative and quantisation settings, the attention back-end switch.  Added:
``max_prefill_chunk`` (a cap on one request's prompt portion in a step, so that decoding
requests ride along with short portions).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .model_config import ModelConfig

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def parse_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in DTYPES.values():
            raise ValueError(f"dtype {dtype} is not supported (bfloat16 or float32)")
        return dtype
    if dtype not in DTYPES:
        raise ValueError(f"dtype {dtype!r} is not supported (bfloat16 or float32)")
    return DTYPES[dtype]


@dataclass
class CacheConfig:
    """Paged cache sizes (src/tokenvault/config.py:75-102).  Either ``num_blocks`` or
    ``kv_cache_memory_gb`` fixes the pool."""

    block_size: int = 16
    num_blocks: int | None = 256
    kv_cache_memory_gb: float | None = None
    # Fraction of blocks kept free at admission so that a new request is not preempted at once.
    watermark: float = 0.01
    dtype: torch.dtype = torch.bfloat16

    def resolve_num_blocks(self, bytes_per_block: int) -> int:
        """src/tokenvault/config.py:97-102, with the bytes of one block (all layers, keys and
        values) given by the cache groups of the model."""
        if self.num_blocks is not None:
            return self.num_blocks
        if self.kv_cache_memory_gb is None:
            raise ValueError("either num_blocks or kv_cache_memory_gb must be set")
        return max(1, math.floor(self.kv_cache_memory_gb * 1024**3 / max(1, bytes_per_block)))


@dataclass
class SchedulerConfig:
    """src/tokenvault/config.py:105-111 (first come, first served only)."""

    max_num_seqs: int = 32
    max_num_batched_tokens: int = 2048
    max_model_len: int = 2048
    enable_chunked_prefill: bool = True
    max_prefill_chunk: int | None = None


@dataclass
class EngineConfig:
    """src/tokenvault/config.py:134-151.  ``model`` may be left ``None`` when the engine is
    given a model folder."""

    model: ModelConfig | None = None
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    device: str = "cuda"
    dtype: torch.dtype = torch.bfloat16
    seed: int = 0
    # Replay single-token batches as CUDA graphs (bfloat16 serving path).
    cuda_graphs: bool = True
    # Read a step's tokens while the next step runs (a decoded token feeds the next step on the
    # device; stop tokens are seen one step late).  False: read them before the next step.
    async_output: bool = True

    def __post_init__(self) -> None:
        self.dtype = parse_dtype(self.dtype)
        self.finalize()

    def finalize(self) -> None:
        if self.model is not None:
            self.scheduler.max_model_len = min(self.scheduler.max_model_len, self.model.max_position_embeddings)
        self.cache.dtype = self.dtype
