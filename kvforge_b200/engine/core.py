"""Everything below the scheduler, put together once: the model built from its spec, its
weights on the device, the page allocator, the state slots, the device pools and the step
function.  ``InferenceEngine`` and the trace-replay program both stand on this, so what is
replayed is what generates.

The order of construction follows umarhassan-cloud/kvforge's ``InferenceEngine.__init__``
(src/tokenvault/engine.py:52-72).
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..cache.block_manager import BlockManager, GroupSpec
from ..cache.kv_pool import KVPool, bytes_per_block
from ..cache.state_slots import StateSlotPool
from ..config.engine_config import CacheConfig, parse_dtype
from ..config.model_config import read_config_json
from ..config.registry import architecture_of, get_architecture
from ..parts.model import DecoderModel, ModelSpec
from ..weights.loader import load_weights
from ..weights.random_init import random_weights
from .runtime import Runtime
from .step import ModelRunner


def spec_from_model_dir(model_dir: str | Path):
    """(typed config, ModelSpec) of a model folder; the class is chosen by ``config.json``."""
    cj = read_config_json(model_dir)
    arch = architecture_of(cj)
    cfg = arch.parse_config(cj)
    return cfg, arch.build_spec(cfg)


def spec_from_config(cfg) -> ModelSpec:
    return get_architecture(cfg.architectures[0]).build_spec(cfg)


class EngineCore:
    def __init__(
        self,
        spec: ModelSpec,
        *,
        dtype: torch.dtype | str,
        device: str = "cuda",
        model_dir: str | Path | None = None,
        seed: int = 0,
        init_std: float = 0.02,
        cache: CacheConfig | None = None,
        max_num_seqs: int = 32,
        max_num_batched_tokens: int = 2048,
        max_model_len: int = 2048,
        cuda_graphs: bool = False,
        lazy_buffers: bool = False,
        pdl: bool | None = None,
    ) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("kvforge_b200 needs a CUDA device: there is no CPU path")
        # The library's bfloat16 products sum in 32-bit, also across slices of K of the library's own
        # choosing (a setting of this process; it costs nothing measurable on the products of this engine).
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.spec = spec
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        self.max_model_len = int(max_model_len)
        cache = cache or CacheConfig()
        self.model = DecoderModel(spec)
        self.rt = Runtime(self.device, self.dtype, max_num_batched_tokens, max_num_seqs, self.max_model_len, lazy=lazy_buffers)
        expected = self.model.expected_weights()
        if model_dir is not None:
            weights = load_weights(model_dir, expected, self.dtype, self.device, spec.ignore_suffixes)
        else:
            skip = (spec.lm_head_name,) if spec.tie_word_embeddings else ()
            weights = random_weights(expected, seed, self.dtype, self.device, init_std=init_std, skip=skip)
        self.model.bind(weights, self.rt)
        del weights

        self.block_size = cache.block_size
        per_block = bytes_per_block(self.model, cache.block_size, self.dtype)
        self.num_blocks = cache.resolve_num_blocks(per_block)
        groups = [GroupSpec(g.need.kind, g.need.window) for g in self.model.groups] or [GroupSpec()]
        self.block_manager = BlockManager(self.num_blocks, cache.block_size, cache.watermark, groups)
        self.state_slots = StateSlotPool(max_num_seqs)
        self.pool = KVPool(self.model, self.num_blocks, cache.block_size, max_num_seqs, self.dtype, self.device)
        self.runner = ModelRunner(
            self.model, self.rt, self.block_manager, self.state_slots, self.max_model_len, cuda_graphs=cuda_graphs,
            pdl=(self.dtype == torch.bfloat16) if pdl is None else pdl,
        )  # fmt: skip
        self.runner.attach_pool(self.pool)

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, **kw) -> EngineCore:
        cfg, spec = spec_from_model_dir(model_dir)
        core = cls(spec, model_dir=model_dir, **kw)
        core.config = cfg
        return core
