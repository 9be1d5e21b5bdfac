"""A decoder as data (``ModelSpec``) and the object that runs it (``DecoderModel``).

The spec names, layer by layer, the block arrangement and the parts in it, and gives the
order in which layers run as a list of ``LayerCall``: a layer may be named twice (it then
has a cache entry per call), and a call may read the keys and values that an earlier call
wrote (``kv_from``) instead of keeping its own.  The step's flow is that of
umarhassan-cloud/kvforge's ``Transformer.forward`` (src/tokenvault/model.py:175-191): embed,
blocks, final norm, and the output head on the wanted rows only
(src/tokenvault/batching/continuous.py:117), logits in 32-bit.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import embedding as _embedding, head as _head  # noqa: F401  (register the default parts)
from .base import Block, CacheNeed, LayerCache, PartSpec, WeightDecl, build_part


@dataclass
class LayerSpec:
    block: PartSpec
    prefix: str  # checkpoint prefix of the layer, e.g. "model.layers.3."


@dataclass
class LayerCall:
    layer: int
    kv_from: int | None = None  # index (in the execution list) of the call whose cache is read


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: list[LayerSpec]
    final_norm: PartSpec
    execution: list[LayerCall] = field(default_factory=list)
    tie_word_embeddings: bool = False
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    lm_head_name: str = "lm_head.weight"
    # names that may be in a checkpoint and are not weights
    ignore_suffixes: tuple[str, ...] = ("rotary_emb.inv_freq",)
    max_position_embeddings: int = 0
    # what turns token ids into the residual stream and normed rows into logits (defaults: the token
    # embedding and the linear head of the model's sizes); their tensors are ``embedding_name`` and
    # ``lm_head_name``
    embedding: PartSpec | None = None
    head: PartSpec | None = None
    # a position encoding that acts on the residual stream after the embedding lookup (``embed``);
    # its tensors, if it has any, carry ``input_position_prefix``
    input_position: PartSpec | None = None
    input_position_prefix: str = "model.embed_positions."
    eos_token_id: int | None = None
    bos_token_id: int | None = None

    def __post_init__(self) -> None:
        if not self.execution:
            self.execution = [LayerCall(i) for i in range(len(self.layers))]
        for idx, call in enumerate(self.execution):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"execution[{idx}] names layer {call.layer}, which does not exist")
            if call.kv_from is not None:
                if not 0 <= call.kv_from < idx:
                    raise ValueError(f"execution[{idx}].kv_from must name an earlier call")
                if self.execution[call.kv_from].kv_from is not None:
                    raise ValueError(f"execution[{idx}].kv_from names a call that keeps no cache of its own")


@dataclass
class CacheGroup:
    """Calls whose mixers keep the same thing per token share pages and a block table."""

    need: CacheNeed
    calls: list[int]  # execution indices that own an entry, in order


class DecoderModel:
    """Builds the parts of a ``ModelSpec``; ``expected_weights`` feeds the loader, ``bind``
    takes the tensors, ``attach_cache`` the pools, ``forward`` runs one step."""

    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.blocks: list[Block] = [build_part("block", ls.block, ls.prefix) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm_prefix)
        sizes = {"vocab_size": spec.vocab_size, "hidden_size": spec.hidden_size}
        for name in (spec.embedding_name, spec.lm_head_name):
            if not name.endswith("weight"):
                raise ValueError(f"tensor name {name!r} must end in 'weight'")
        self.embedding = build_part("embedding", spec.embedding or PartSpec("token_embedding", sizes), spec.embedding_name[: -len("weight")])
        self.head = build_part("head", spec.head or PartSpec("linear_head", sizes), spec.lm_head_name[: -len("weight")])
        self.input_position = build_part("position", spec.input_position, spec.input_position_prefix) if spec.input_position else None
        # cache groups from what the mixers declare
        self.groups: list[CacheGroup] = []
        self.call_group: list[tuple[int, int] | None] = []  # per call: (group, entry) of its own cache
        for idx, call in enumerate(spec.execution):
            mixer = self.blocks[call.layer].mixer_part()
            need = mixer.cache_need() if mixer is not None else CacheNeed("none")
            if call.kv_from is not None or need.kind == "none":
                self.call_group.append(None)
                continue
            for gi, g in enumerate(self.groups):
                if g.need.group_key == need.group_key:
                    g.calls.append(idx)
                    self.call_group.append((gi, len(g.calls) - 1))
                    break
            else:
                self.groups.append(CacheGroup(need, [idx]))
                self.call_group.append((len(self.groups) - 1, 0))
        for idx, call in enumerate(spec.execution):
            if call.kv_from is not None:
                src = spec.execution[call.kv_from]
                a = self.blocks[call.layer].mixer_part().cache_need()
                b = self.blocks[src.layer].mixer_part().cache_need()
                if a.group_key != b.group_key:
                    raise ValueError(f"execution[{idx}] reads a cache of another shape than its mixer's")
        self.state_shapes: list[tuple[int, ...] | None] = []
        for call in spec.execution:
            mixer = self.blocks[call.layer].mixer_part()
            self.state_shapes.append(mixer.state_shape() if mixer is not None else None)
        self.caches: list[LayerCache | None] = [None] * len(spec.execution)

    # ------------------------------------------------------------------ weights
    def expected_weights(self) -> dict[str, WeightDecl]:
        """Checkpoint tensor name -> declaration, for everything the model needs."""
        out: dict[str, WeightDecl] = {}
        for part in self._all_parts():
            for local, decl in type(part).weight_decls(part.params).items():
                out[part.prefix + local] = decl
        return out

    def _all_parts(self):
        yield self.embedding
        yield self.head
        for block in self.blocks:
            yield from block.sub_parts()
        yield self.final_norm
        if self.input_position is not None:
            yield self.input_position

    def bind(self, weights: dict[str, torch.Tensor], rt) -> None:
        s = self.spec
        self.rt = rt
        shared_positions: dict[str, object] = {}
        for part in self._all_parts():
            pos_spec = getattr(part, "position_spec", None)
            if pos_spec is not None:
                key = pos_spec.key()
                if key not in shared_positions:
                    inst = build_part("position", pos_spec)
                    inst.bind({}, rt)
                    shared_positions[key] = inst
                part.position = shared_positions[key]
            local = {name: weights[part.prefix + name] for name in type(part).weight_decls(part.params) if part.prefix + name in weights}
            part.bind(local, rt)
        # kvforge: one tensor when tied, and the embedding stands in when the head is absent
        # (src/tokenvault/model.py:157-158, src/tokenvault/model_loader.py:105-106)
        if s.tie_word_embeddings or s.lm_head_name not in weights:
            self.head.tie(self.embedding.table())

    def attach_cache(self, caches: list[LayerCache | None]) -> None:
        """``caches[i]`` is what call ``i`` of the execution list reads and writes."""
        if len(caches) != len(self.spec.execution):
            raise ValueError("one cache entry per call of the execution list is needed")
        self.caches = list(caches)

    # ------------------------------------------------------------------ step
    def forward_hidden(self, ctx):
        """Runs the blocks.  Returns the float residual stream and the sum still pending."""
        rt = self.rt
        resid = rt.buf("model.resid", ctx.num_tokens, self.spec.hidden_size, torch.float32)
        self.embedding.forward(ctx, resid)
        ctx.residual = resid
        if self.input_position is not None:
            self.input_position.embed(ctx, resid)
        delta = None
        for idx, call in enumerate(self.spec.execution):
            delta = self.blocks[call.layer].forward(ctx, resid, delta, self.caches[idx])
        return resid, delta

    def forward(self, ctx) -> torch.Tensor:
        """Float logits ``[R, vocab]`` at ``ctx.logit_rows``."""
        rt = self.rt
        resid, delta = self.forward_hidden(ctx)
        r = ctx.num_logit_rows
        if r == 0:
            return rt.buf("model.logits", 0, self.spec.vocab_size, torch.float32, cap=rt.max_seqs)
        x = self.final_norm.forward(ctx, resid, delta, rows=ctx.logit_rows, num_rows=r)
        return self.head.forward(ctx, x)
