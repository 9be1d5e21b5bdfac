"""Grouped-query attention over the paged cache (the mixer of the Llama decoder).

What it computes is umarhassan-cloud/kvforge's ``Attention.forward``
(src/tokenvault/model.py:77-92): bias-free q/k/v projections, rotation of q and k, the step's
k and v written to their slots *before* attention reads the cache, causal attention over
the block table (src/tokenvault/cache/paged_attention.py:66-91), output projection.
The three input projections are one product here (their weights are stacked at load).
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import CacheNeed, Mixer, PartSpec, WeightDecl, build_part, register_mixer
from .projection import PART_ROWS, project


# Decode attention merges its key ranges through a thread-block cluster's shared memory only with
# this few (sequence, kv head) pairs: measured inside the decode step it gains 2 % at one sequence
# and loses at 8 and 64, where the ranges past the context (a captured graph's grid covers twice
# the context at most) hold their places until their cluster is done.
CLUSTER_MERGE_MAX_PAIRS = 16

@register_mixer("paged_attention")
class PagedAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``; optional
    ``position`` (a position-encoding ``PartSpec`` or ``None``), ``window`` (keys a query
    sees, itself included; ``None`` = all) and ``scale`` (default ``1/sqrt(head_dim)``)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.nh = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        ops.check_head_dim(self.d)
        self.window = params.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("window must be positive")
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.d))  # model.py:74
        pos = params.get("position")
        if isinstance(pos, dict):
            pos = PartSpec(pos["kind"], pos.get("params", {}))
        self.position_spec: PartSpec | None = pos
        self.position = None  # shared instance, set by the model before bind
        self.q_dim = self.nh * self.d
        self.qkv_dim = (self.nh + 2 * self.nkv) * self.d

    @classmethod
    def weight_decls(cls, params):
        h, nh, nkv, d = (int(params[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        return {
            "q_proj.weight": WeightDecl((nh * d, h)),
            "k_proj.weight": WeightDecl((nkv * d, h)),
            "v_proj.weight": WeightDecl((nkv * d, h)),
            "o_proj.weight": WeightDecl((h, nh * d)),
        }

    def cache_need(self) -> CacheNeed:
        if self.window is None:
            return CacheNeed("full", self.nkv, self.d, None)
        return CacheNeed("window", self.nkv, self.d, int(self.window))

    def bind(self, weights, rt):
        super().bind(weights, rt)
        self.w_qkv = torch.cat([weights["q_proj.weight"], weights["k_proj.weight"], weights["v_proj.weight"]], dim=0).contiguous()
        self.w_o = weights["o_proj.weight"].contiguous()
        # counters of finished key ranges per (sequence, kv head) for the decode form: zero between launches
        self._tickets = torch.zeros(max(1, rt.max_seqs) * self.nkv, dtype=torch.int32, device=rt.device)
        # the kernel of prompts and mixed batches takes its tiles of queries from a list made with the step
        self._query_tile = None
        if ops.tcgen05_attention_supported(rt.dtype, self.nh, self.nkv, self.d, False):
            self._query_tile = ops.tcgen05_query_tile(self.nh, self.nkv)
            rt.query_tile_sizes.add(self._query_tile)
        if self.position_spec is not None and self.position is None:
            self.position = build_part("position", self.position_spec)
            self.position.bind({}, rt)
        table = self.position.table() if self.position is not None else None
        # no table: q and k are stored and used as the projections leave them
        self.inv_freq = table if table is not None else torch.empty(0, dtype=torch.float32, device=rt.device)

    def _scratch(self, ctx):
        rt = self.rt
        # buffers are made for the longest context the engine takes; the grid follows the longest
        # context of this step (of this graph, when the step is captured)
        bound = max(ctx.context_bound, ctx.max_context_len, rt.max_model_len, 1)
        reach = max(ctx.context_bound if ctx.context_bound > 0 else ctx.max_context_len, 1)
        # 32-bit: one range size whatever the batch, so a request's sums come in the same order beside
        # any number of others; bfloat16: longer ranges for many sequences (fewer CTAs, same bytes)
        split = ops.attention_split_size(ctx.num_seqs if rt.dtype == torch.bfloat16 else 1, self.nkv, bound, reach, self.d)
        # made for the smallest range size, so that one buffer serves every batch size
        smallest = min(ops.attention_split_size(1, 1, bound), ops.attention_split_size(ops.ATTN_SHORT_RANGE_PAIRS[0], 1, bound))
        sa, sm = ops.attention_scratch_shapes(max(rt.max_seqs, ctx.num_seqs), self.nh, self.d, bound, smallest)
        acc = rt.buf("attn.part_acc", sa[0] * sa[1] * sa[2], sa[3], torch.float32, cap=0).view(sa)
        ml = rt.buf("attn.part_ml", sm[0] * sm[1] * sm[2], sm[3], torch.float32, cap=0).view(sm)
        if self._tickets.numel() < sa[0] * self.nkv:
            if rt.capturing or rt.graphs_captured:
                raise RuntimeError("the attention tickets would have to grow after or during graph capture")
            self._tickets = torch.zeros(sa[0] * self.nkv, dtype=torch.int32, device=rt.device)
        return (acc, ml, self._tickets), reach, split

    def forward(self, ctx, x: torch.Tensor, cache) -> torch.Tensor:
        rt = self.rt
        n = x.shape[0]
        if cache is None:
            raise RuntimeError("paged_attention needs a cache")
        skinny = ops.skinny_ok(x, self.w_qkv)
        if cache.writable:
            slots = ctx.slot_mappings[cache.group]
            splits = ops.skinny_splits(self.qkv_dim, self.hidden, n) if skinny else 1
            if splits > 1:
                # decode: slices of K in parallel; the rotation kernel sums them
                part = ops.Partials(rt.buf("attn.qkv_part", splits * n, self.qkv_dim, torch.float32, cap=PART_ROWS).view(splits, n, self.qkv_dim))
                ops.gemm_skinny(x, self.w_qkv, part)
                q = rt.buf("attn.q", n, self.q_dim)
                ops.rope_cache_write(part, ctx.positions, self.inv_freq, slots, cache.k, cache.v, self.nh, self.nkv, self.d, ctx.block_size, rt.err, q_out=q)
                q_stride = self.q_dim
            else:
                qkv = rt.buf("attn.qkv", n, self.qkv_dim)
                if skinny:
                    ops.gemm_skinny(x, self.w_qkv, qkv)
                else:
                    ops.linear(x, self.w_qkv, qkv)
                ops.rope_cache_write(qkv, ctx.positions, self.inv_freq, slots, cache.k, cache.v, self.nh, self.nkv, self.d, ctx.block_size, rt.err)
                q, q_stride = qkv, self.qkv_dim
        else:
            # reads another call's keys and values: only the queries are needed
            q = rt.buf("attn.q", n, self.q_dim)
            ops.linear(x, self.w_qkv[: self.q_dim], q)
            ops.rope_cache_write(q, ctx.positions, self.inv_freq, None, None, None, self.nh, 0, self.d, ctx.block_size)
            q_stride = self.q_dim
        out = rt.buf("attn.out", n, self.q_dim)
        self.attend(ctx, q, q_stride, out, cache)
        return project(rt, "attn.proj", out, self.w_o, ctx)

    def attend(self, ctx, q, q_stride, out, cache) -> None:
        scratch, bound, split = None, None, 256
        common = dict(window=int(self.window or 0), q_stride=q_stride, err=self.rt.err)
        args = (q, out, cache.k, cache.v, ctx.block_tables[cache.group], ctx.query_start_loc, ctx.context_lens, ctx.num_seqs)
        shape = (self.nh, self.nkv, self.d, self.scale)
        # bfloat16: the decode kernel may lengthen its key ranges from the step's longest context (the merge
        # order then follows the batch, within rounding); 32-bit keeps one order whatever the batch
        wave = ops.attention_wave_target(ctx.num_seqs, self.nkv, self.d) if q.dtype == torch.bfloat16 else 0
        if ctx.all_single_query:
            scratch, bound, split = self._scratch(ctx)
        tiles = ctx.query_tiles.get(self._query_tile)
        if tiles is not None and tiles.num_single > 0 and ops.tma_decode_supported(q.dtype, self.nh, self.nkv, self.d, ctx.block_size, cache.k.shape[0]):
            # a mixed batch: the sequences that bring one token go to the decode kernel (key ranges in
            # parallel), the portions of prompts to the kernel of prompts; each leaves the other's rows alone
            scratch, bound, split = self._scratch(ctx)
            side = self.rt.side_stream() if (self.rt.capturing and tiles.multi_count > 0) else None
            if side is not None:
                # the two kernels write other rows, and one is bound by the tensor cores, the other by memory: in
                # a captured step they are two branches that run side by side (32 decoding requests beside a
                # 1,024-token portion: 2.98 -> 2.86 ms at the 1B shape, 7.86 -> 7.58 ms at the 3B shape)
                main = torch.cuda.current_stream()
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    ops.paged_attention(*args, ctx.max_query_len, *shape, query_tiles=(tiles.multi, tiles.multi_count), **common)
            ops.paged_attention(*args, 1, *shape, scratch=scratch, max_context=bound, split_size=split, kernel="tma", cluster=False, single_only=True, wave_target=wave, **common)
            if side is not None:
                torch.cuda.current_stream().wait_stream(side)
            elif tiles.multi_count > 0:
                ops.paged_attention(*args, ctx.max_query_len, *shape, query_tiles=(tiles.multi, tiles.multi_count), **common)
            return
        ops.paged_attention(
            *args, ctx.max_query_len, *shape, scratch=scratch, max_context=bound, split_size=split,
            cluster=ctx.num_seqs * self.nkv <= CLUSTER_MERGE_MAX_PAIRS, wave_target=wave if scratch is not None else 0,
            query_tiles=(tiles.tiles, tiles.count) if tiles is not None else None, **common,
        )  # fmt: skip
