"""The parts a model is put together from.  Importing the package registers the built-in
ones (token embedding, rotary encoding, RMSNorm, paged attention, gated feed-forward, pre-norm
block, linear head)."""

from . import attention, block, embedding, head, mlp, norm, rope  # noqa: F401  (registration)
from .base import (  # noqa: F401
    CacheNeed,
    LayerCache,
    PartSpec,
    WeightDecl,
    register_block,
    register_embedding,
    register_feed_forward,
    register_head,
    register_mixer,
    register_norm,
    register_position_encoding,
)
from .model import DecoderModel, LayerCall, LayerSpec, ModelSpec  # noqa: F401
