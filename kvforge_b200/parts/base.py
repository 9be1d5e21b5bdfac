"""Interfaces of the parts a model is put together from, and their registries.

A part is built from a ``PartSpec`` (a registry name and a dict of sizes and constants)
and a weight-name prefix.  It says which tensors it needs (``weight_decls``), is handed
them (``bind``) and is then run with a ``StepContext``.  No part knows which model it is
in, which layer it is, or what the other parts are; what it needs of the batch it takes
from the context, what it needs of the cache from the view it is given.

Kinds of part and the call each must answer:

* position encoding — either of two calls, each with a default that does nothing.
  ``table()`` is for encodings that turn pairs of query and key dims by the token's position:
  it returns the float frequencies ``[rot/2]`` that the mixer's kernel multiplies positions
  with (``None``: queries and keys are left as they are).  Such an encoding is named in a
  mixer's ``position`` parameter, built once per distinct spec and shared.
  ``embed(ctx, resid)`` is for encodings that act on the residual stream right after the
  embedding lookup (learned or fixed absolute positions): it adds to ``resid[n]`` in place from
  ``ctx.positions``.  Such an encoding is named in ``ModelSpec.input_position`` and may have
  weights of its own.
* norm — ``forward(ctx, resid, delta, rows=None) -> x``: adds ``delta`` (``None``, a tensor in
  the storage type, the ``ops.Partials`` of a split-K product, or ``ops.ADDED`` when its
  producer has added it into ``ctx.residual`` already) into the float residual stream, returns
  the normed rows in the storage type.
* mixer — ``cache_need()`` and ``state_shape()`` declare what it keeps between steps;
  ``forward(ctx, x, cache) -> y`` mixes along the sequence.  ``cache`` is a
  ``LayerCache`` (pages of this call, or of the call it reads) or ``None``.  ``y`` is a
  tensor in the storage type, ``ops.Partials`` or ``ops.ADDED``; only a norm ever reads it.
* feed-forward — ``forward(ctx, x) -> y`` per token (``y`` as for a mixer).
* embedding — ``forward(ctx, resid)`` fills the float residual stream ``[N, hidden]`` from the
  step's token ids (``ctx.token_ids``, or where ``ctx.feedback_rows[n] >= 0`` the token the
  device sampled a step before: ``ctx.token_feedback[ctx.feedback_rows[n]]``); ``table()``
  returns its ``[vocab, hidden]`` tensor for a head that shares it.
* head — ``forward(ctx, x) -> logits``: float logits ``[R, vocab]`` of the ``R`` normed rows it is
  given; ``tie(table)`` hands it the embedding's tensor when the model ties the two or the
  checkpoint has no tensor for it.
* block — the arrangement of the above in one layer:
  ``forward(ctx, resid, delta, cache) -> delta`` (the sum not yet added to ``resid``).  An
  arrangement in which a part's result must not go straight into the residual stream (a norm
  after the sum, two parts reading the same stream) sets ``ctx.residual = None`` around that
  part's call and gets a tensor or ``ops.Partials`` back.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class WeightDecl:
    """One tensor a part needs.  ``kind``: ``matrix`` (held in the storage type), ``vector``
    (held in float: a 32-bit tensor stays 32-bit, a 16-bit one is widened exactly) or
    ``table`` (integers, held as int32).  ``init`` is how the random-weights mode fills it."""

    shape: tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per token.  ``kind``: ``full`` (every key), ``window`` (the last
    ``window`` keys) or ``none``."""

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None

    @property
    def group_key(self) -> tuple:
        return (self.kind, self.kv_heads, self.head_dim, self.window)


@dataclass
class PartSpec:
    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def key(self) -> str:
        return f"{self.kind}:{sorted((k, repr(v)) for k, v in self.params.items())}"


@dataclass
class LayerCache:
    """The pages one mixer call reads and, if ``writable``, writes."""

    k: torch.Tensor  # [num_blocks, kv_heads, block_size, head_dim]
    v: torch.Tensor
    group: int  # index of the cache group: selects the block table and slots in the context
    writable: bool = True
    state: torch.Tensor | None = None  # [num_slots, *state_shape] if the mixer has state


class Part:
    """Base of every part."""

    def __init__(self, params: dict[str, Any], prefix: str = "") -> None:
        self.params = dict(params)
        self.prefix = prefix

    @classmethod
    def weight_decls(cls, params: dict[str, Any]) -> dict[str, WeightDecl]:
        """Local tensor name -> declaration.  The checkpoint name is ``prefix + local``."""
        return {}

    def bind(self, weights: dict[str, torch.Tensor], rt: Any) -> None:
        """Take the device tensors (keyed by local name) and whatever else the run needs."""
        self.rt = rt


class PositionEncoding(Part):
    def table(self) -> torch.Tensor | None:
        """Float frequencies ``[rot/2]`` for a mixer that turns q and k, or ``None``."""
        return None

    def embed(self, ctx, resid: torch.Tensor) -> None:
        """Add this encoding to the float residual stream after the embedding lookup."""
        return None


class Norm(Part):
    def forward(self, ctx, resid, delta, rows=None):  # pragma: no cover - interface
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return CacheNeed("none")

    def state_shape(self) -> tuple[int, ...] | None:
        """Shape of the fixed-size float state per request, or ``None``."""
        return None

    def forward(self, ctx, x, cache):  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x):  # pragma: no cover - interface
        raise NotImplementedError


class Embedding(Part):
    def table(self) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def forward(self, ctx, resid: torch.Tensor) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class Head(Part):
    def tie(self, table: torch.Tensor) -> None:  # pragma: no cover - interface
        raise NotImplementedError

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError


class Block(Part):
    """Arrangement of parts in a layer.  Sub-parts are built from ``params`` by ``build_part``."""

    def sub_parts(self) -> list[Part]:
        return []

    def mixer_part(self) -> Mixer | None:
        return None

    def forward(self, ctx, resid, delta, cache):  # pragma: no cover - interface
        raise NotImplementedError


# ------------------------------------------------------------------ registries

POSITION_ENCODINGS: dict[str, type[PositionEncoding]] = {}
NORMS: dict[str, type[Norm]] = {}
MIXERS: dict[str, type[Mixer]] = {}
FEED_FORWARDS: dict[str, type[FeedForward]] = {}
BLOCKS: dict[str, type[Block]] = {}
EMBEDDINGS: dict[str, type[Embedding]] = {}
HEADS: dict[str, type[Head]] = {}

_FAMILIES = {
    "position": POSITION_ENCODINGS,
    "norm": NORMS,
    "mixer": MIXERS,
    "ffn": FEED_FORWARDS,
    "block": BLOCKS,
    "embedding": EMBEDDINGS,
    "head": HEADS,
}


def _register(family: str, name: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        table = _FAMILIES[family]
        if name in table and table[name] is not cls:
            raise ValueError(f"{family} part {name!r} is already registered")
        table[name] = cls
        cls.kind = name
        return cls

    return deco


def register_position_encoding(name: str):
    return _register("position", name)


def register_norm(name: str):
    return _register("norm", name)


def register_mixer(name: str):
    return _register("mixer", name)


def register_feed_forward(name: str):
    return _register("ffn", name)


def register_block(name: str):
    return _register("block", name)


def register_embedding(name: str):
    return _register("embedding", name)


def register_head(name: str):
    return _register("head", name)


def build_part(family: str, spec: PartSpec, prefix: str = "") -> Part:
    table = _FAMILIES[family]
    if spec.kind not in table:
        raise KeyError(f"no {family} part named {spec.kind!r} (known: {sorted(table)})")
    return table[spec.kind](spec.params, prefix)
