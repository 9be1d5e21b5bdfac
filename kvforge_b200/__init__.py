"""kvforge_b200: a small, whole inference engine for the dense Llama decoder on one B200.

From a model folder (``config.json`` + safetensors) or seeded random weights to generated
tokens: typed configuration and an architecture registry, a loader by tensor name, a model
put together from parts, a paged cache with block tables, one step function for flat
batches of prompt portions and decoded tokens, a token-budget scheduler, sampling on the
device, all on hand-written CUDA kernels for sm_100a (in bfloat16 and in true float32).
"""

import os as _os

# The library's matrix products inside a captured step get the workspace that cuBLASLt is given
# when it is first used; with torch's default (1 MiB) the products of a 2,048-token step at the
# widths of Llama-3.1-8B run 5 % slower captured than launched one by one.  64 MiB (the unit is
# KiB) unless the caller has said otherwise.
_os.environ.setdefault("CUBLASLT_WORKSPACE_SIZE", "65536")

from .config.engine_config import CacheConfig, EngineConfig, SchedulerConfig  # noqa: E402
from .config.model_config import ConfigError, ModelConfig, RopeScaling
from .config.registry import PRESETS, register_architecture
from .engine.request import FinishReason, Request, RequestOutput, RequestStatus
from .sampling.params import SamplingParams

__version__ = "0.1.0"

__all__ = [
    "PRESETS",
    "CacheConfig",
    "ConfigError",
    "EngineConfig",
    "FinishReason",
    "InferenceEngine",
    "ModelConfig",
    "Request",
    "RequestOutput",
    "RequestStatus",
    "RopeScaling",
    "SamplingParams",
    "SchedulerConfig",
    "ByteTokenizer",
    "register_architecture",
    "write_random_model",
    "__version__",
]


def __getattr__(name):
    # The engine pulls in the parts and the native loader; keep `import kvforge_b200` light.
    if name == "InferenceEngine":
        from .engine.engine import InferenceEngine

        return InferenceEngine
    if name == "ByteTokenizer":
        from .engine.tokenizer import ByteTokenizer

        return ByteTokenizer
    if name == "write_random_model":
        from .models.folder import write_random_model

        return write_random_model
    raise AttributeError(name)
