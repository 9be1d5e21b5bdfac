"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

Same contract as umarhassan-cloud/kvforge's ``prepare_inputs`` + ``ModelRunner.execute``
(src/tokenvault/batching/continuous.py:44-117): items are whole prompts, portions of prompts
at any start position, or single decoded tokens, mixed freely; all of them run as one flat
batch; only the tokens given are computed, everything before them comes from the cache;
pages for the new positions must have been reserved by the caller.

Different in how: all index arrays are int32 and are packed on the host into one pinned
buffer that goes to the device in a single copy; the device copy lives at fixed addresses.
A step of single tokens only is, per batch-size bucket, captured once as a CUDA graph and
replayed (the arrays it reads are then laid out for the bucket's full width, so the
addresses inside the graph stay valid); so is a step of many tokens, for its token count
rounded up, from the second time its shape comes.  Beside the arrays that umarhassan-cloud/kvforge
prepares, a step carries lists of its tiles of queries (sequence, first query) for kernels that
take a fixed number of queries of one sequence per CTA.
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
from ..cache.block_manager import BlockManager
from ..cache.state_slots import StateSlotPool
from .runtime import QueryTiles, Runtime, StepContext


# graphs for shorter contexts than this are not told apart
MIN_GRAPH_CONTEXT = 1024
# steps of at least this many tokens (more than the decode GEMM takes) are replayed as graphs too, padded to a
# multiple of GRAPH_TOKEN_STEP: a few decoding requests beside a short portion of a prompt are some 150 kernels,
# which take longer to launch from Python than to run
# (padding is work: 224 tokens beside 1,056 cost a fifth more); a shape is captured the second time it comes
MIN_GRAPH_TOKENS = 17
GRAPH_TOKEN_STEP = 64


@dataclass
class BatchItem:
    """``logits``: ``"last"``, ``"all"``, ``"none"`` (continuous.py:24-32) or a list of places
    among ``token_ids`` whose logits are wanted."""

    seq_id: str
    token_ids: Sequence[int]
    start_pos: int
    logits: str | Sequence[int] = "last"
    # For a single token that the device sampled in the step before and the host has not read
    # yet: its row in the runner's ``token_feedback`` buffer (``token_ids`` is then ignored).
    feedback_row: int | None = None

    def wanted(self) -> list[int]:
        n = len(self.token_ids)
        if isinstance(self.logits, str):
            if self.logits == "last":
                return [n - 1]
            if self.logits == "all":
                return list(range(n))
            if self.logits == "none":
                return []
            raise ValueError(f"logits mode {self.logits!r}")
        out = [int(i) for i in self.logits]
        for i in out:
            if not 0 <= i < n:
                raise ValueError(f"wanted place {i} is outside the {n} tokens of {self.seq_id}")
        return out


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


@dataclass
class _Layout:
    """Offsets (in int32 elements) of the arrays of a step inside the metadata buffer."""

    n_cap: int
    b_cap: int
    width: int
    n_groups: int
    r_cap: int
    tile_sizes: tuple[int, ...] = ()
    off: dict[str, int] = field(default_factory=dict)
    total: int = 0

    def __post_init__(self) -> None:
        o = 0
        for name, size in (
            ("token_ids", self.n_cap),
            ("positions", self.n_cap),
            ("feedback_rows", self.n_cap),
            ("logit_rows", self.r_cap),
            ("qsl", self.b_cap + 1),
            ("ctx", self.b_cap),
            ("state_slots", self.b_cap),
            ("slots", self.n_groups * self.n_cap),
            ("tables", self.n_groups * self.b_cap * self.width),
        ):
            self.off[name] = o
            o += _align(size)
        for tq in self.tile_sizes:  # pairs (sequence, first query) per tile of tq queries: all, and without single tokens
            for name in (f"qtiles_{tq}", f"qtiles_multi_{tq}"):
                self.off[name] = o
                o += _align(2 * self.tile_cap(tq))
        self.total = o

    def tile_cap(self, tq: int) -> int:
        """The most tiles of ``tq`` queries that ``n_cap`` tokens in ``b_cap`` sequences can make."""
        return self.n_cap // tq + self.b_cap


class ModelRunner:
    """Owns the device metadata buffer and runs ``model.forward`` on batches."""

    def __init__(
        self,
        model,
        rt: Runtime,
        block_manager: BlockManager,
        state_slots: StateSlotPool | None,
        max_model_len: int,
        cuda_graphs: bool = False,
        graph_buckets: Sequence[int] = (1, 2, 4, 8, 16, 32, 64, 128, 256),
        pdl: bool = False,
    ) -> None:
        self.model = model
        self.rt = rt
        self.block_manager = block_manager
        self.state_slots = state_slots
        self.block_size = block_manager.block_size
        self.max_model_len = int(max_model_len)
        self.max_width = max(1, -(-self.max_model_len // self.block_size))
        self.n_groups = block_manager.num_groups
        self.cuda_graphs = bool(cuda_graphs)
        self.pdl = bool(pdl)  # programmatic dependent launch between the kernels of a step
        # the most sequences a step can hold is a bucket of its own, so that no batch size goes without a graph
        self.graph_buckets = sorted({b for b in graph_buckets if b <= rt.max_seqs} | ({rt.max_seqs} if rt.max_seqs <= max(graph_buckets) else set())) or [rt.max_seqs]
        # keyed by (tokens, sequences, longest context the graph reaches, single-token sequences in a step of
        # many tokens, decode form); the form is part of the key because a step of many tokens padded to as many
        # tokens as sequences (64 tokens in 64 sequences) is another graph than 64 decoding sequences
        self._graphs: dict[tuple, tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}
        self.graph_kernels: dict[tuple, int] = {}  # kernels of this library inside each captured graph
        self.num_kernel_launches = 0  # kernels of this library launched by steps, replays included
        self.num_graph_kernels = 0  # those of them that ran inside replayed graphs
        self.h2d_bytes = 0  # bytes of step metadata copied to the device so far
        self._cap = 0
        self._host: torch.Tensor | None = None
        self._dev: torch.Tensor | None = None
        self._copy_done: torch.cuda.Event | None = None
        self._tile_counts: dict[int, tuple[int, int, int]] = {}
        self._graph_seen: dict[tuple, int] = {}  # how often a shape of many tokens has come
        self.graph_after = 2  # ... and at which coming it is captured
        # made once for the widest step there can be, so its address never changes
        self._ensure(self._layout(rt.max_tokens, rt.max_seqs, self.max_width, rt.max_tokens).total)
        # tokens sampled on the device that may feed the next step (set by whoever samples)
        self.token_feedback: torch.Tensor | None = None
        self.num_forward_passes = 0  # continuous.py:105-106
        self.num_tokens_processed = 0

    # ------------------------------------------------------------------ buffers
    def _layout(self, n_cap: int, b_cap: int, width: int, r_cap: int) -> _Layout:
        return _Layout(n_cap, b_cap, max(1, width), self.n_groups, max(1, r_cap), tuple(sorted(self.rt.query_tile_sizes)))

    def _ensure(self, total: int) -> None:
        if total <= self._cap:
            return
        if self._graphs:
            raise RuntimeError("the metadata buffer would have to move after graphs were captured")
        self._cap = int(total) + 64
        self._host = torch.empty(self._cap, dtype=torch.int32, pin_memory=True)
        self._dev = torch.empty(self._cap, dtype=torch.int32, device=self.rt.device)

    # ------------------------------------------------------------------ batch building
    def _upload(self, total: int) -> None:
        """The one host-to-device copy of a step."""
        self._dev[:total].copy_(self._host[:total], non_blocking=True)
        self.h2d_bytes += 4 * total
        if self._copy_done is None:
            self._copy_done = torch.cuda.Event()
        self._copy_done.record()

    def _fill(self, items: Sequence[BatchItem], lay: _Layout, padded: bool = False, tiles: bool | None = None) -> tuple[int, int, int, int, int]:
        """Write the arrays of ``items`` into the host buffer under layout ``lay``.

        ``padded``: the layout is wider than the items (a captured shape), so the rest is filled
        first with padding: token 0 at position 0, written to no slot (-1), part of no sequence.
        A padding sequence has no queries (``qsl[b+1] == qsl[b]``), no context and state slot -1;
        a part that keeps state must leave a sequence without queries alone.
        ``tiles``: whether the lists of query tiles are written; by default only when some
        sequence brings more than one token (a step of single tokens launches no kernel that
        reads them).  A captured step of many tokens always launches such a kernel, so its lists
        are written whatever the items."""
        if self._copy_done is not None:
            self._copy_done.synchronize()  # the last step's copy has left the host buffer
        host = self._host.numpy()
        bm, bs = self.block_manager, self.block_size
        o = lay.off
        if padded:
            host[o["token_ids"] : o["token_ids"] + lay.n_cap] = 0
            host[o["positions"] : o["positions"] + lay.n_cap] = 0
            host[o["feedback_rows"] : o["feedback_rows"] + lay.n_cap] = -1
            host[o["logit_rows"] : o["logit_rows"] + lay.r_cap] = 0
            host[o["slots"] : o["slots"] + self.n_groups * lay.n_cap] = -1
        n = 0
        rows: list[int] = []
        max_q = max_ctx = 0
        qsl = host[o["qsl"] : o["qsl"] + lay.b_cap + 1]
        ctx = host[o["ctx"] : o["ctx"] + lay.b_cap]
        sslots = host[o["state_slots"] : o["state_slots"] + lay.b_cap]
        qsl[0] = 0
        for b, item in enumerate(items):
            k = len(item.token_ids)
            if k == 0:
                raise ValueError(f"request {item.seq_id} brings no tokens")
            end = item.start_pos + k
            if end > self.max_model_len:
                raise ValueError(f"request {item.seq_id} would reach {end} tokens, beyond max_model_len {self.max_model_len}")
            if item.feedback_row is None:
                host[o["token_ids"] + n : o["token_ids"] + n + k] = item.token_ids
                host[o["feedback_rows"] + n : o["feedback_rows"] + n + k] = -1
            else:
                if k != 1 or self.token_feedback is None:
                    raise ValueError("a token fed back on the device must be a single token, and a feedback buffer must be set")
                host[o["token_ids"] + n] = 0
                host[o["feedback_rows"] + n] = item.feedback_row
            host[o["positions"] + n : o["positions"] + n + k] = np.arange(item.start_pos, end, dtype=np.int32)
            for g in range(self.n_groups):
                base = o["slots"] + g * lay.n_cap + n
                host[base : base + k] = bm.slots_array(item.seq_id, item.start_pos, end, g)
                table = bm.get_block_table(item.seq_id, g)
                used = -(-end // bs)  # only the pages that cover the live context (continuous.py:67)
                tb = o["tables"] + (g * lay.b_cap + b) * lay.width
                host[tb : tb + used] = table[:used]  # entries past the context are never read
            rows.extend(n + i for i in item.wanted())
            n += k
            qsl[b + 1] = n
            ctx[b] = end
            sslots[b] = self.state_slots.slot(item.seq_id) if (self.state_slots and self.state_slots.has(item.seq_id)) else -1
            max_q = max(max_q, k)
            max_ctx = max(max_ctx, end)
        nb = len(items)
        # padding sequences of a captured bucket: no queries, no context
        for b in range(nb, lay.b_cap):
            qsl[b + 1] = n
            ctx[b] = 0
            sslots[b] = -1
        if len(rows) > lay.r_cap:
            raise RuntimeError("more logit rows than the layout holds")
        host[o["logit_rows"] : o["logit_rows"] + len(rows)] = rows
        if tiles is None:
            tiles = max_q > 1
        self._tile_counts = self._fill_query_tiles(host, lay, nb) if tiles else {}
        return n, nb, len(rows), max_q, max_ctx

    def _fill_query_tiles(self, host: np.ndarray, lay: _Layout, nb: int) -> dict[int, tuple[int, int, int]]:
        """For every registered tile size the step's tiles of queries as (sequence, first query),
        the one with the longest walk over the keys first: once for all sequences, once without
        those that bring a single token.  Returns (tiles, tiles without single tokens, sequences
        with a single token) per size."""
        o = lay.off
        starts = host[o["qsl"] : o["qsl"] + nb + 1].astype(np.int64)
        q_lens = starts[1:] - starts[:-1]
        ctx = host[o["ctx"] : o["ctx"] + nb].astype(np.int64)
        counts: dict[int, tuple[int, int, int]] = {}
        for tq in lay.tile_sizes:
            cap = lay.tile_cap(tq)
            per_seq = -(-q_lens // tq)
            total = int(per_seq.sum())
            seq = np.repeat(np.arange(nb), per_seq)
            q0 = (np.arange(total) - np.repeat(np.cumsum(per_seq) - per_seq, per_seq)) * tq
            last_key = ctx[seq] - q_lens[seq] + np.minimum(q_lens[seq], q0 + tq)
            order = np.argsort(-last_key, kind="stable")
            seq, q0 = seq[order], q0[order]
            multi = q_lens[seq] > 1
            n_multi = int(multi.sum())
            for name, s_, q_, n_ in ((f"qtiles_{tq}", seq, q0, total), (f"qtiles_multi_{tq}", seq[multi], q0[multi], n_multi)):
                tiles = host[o[name] : o[name] + 2 * cap].reshape(cap, 2)
                tiles[:n_, 0] = s_
                tiles[:n_, 1] = q_
                tiles[n_:, 0] = -1
                tiles[n_:, 1] = 0
            counts[tq] = (total, n_multi, int((q_lens == 1).sum()))
        return counts

    def _context(self, lay: _Layout, n: int, nb: int, r: int, max_q: int, max_ctx: int, bound: int, all_tiles: bool = False, singles: bool = True) -> StepContext:
        dev, host, o = self._dev, self._host.numpy(), lay.off
        # a captured step launches every tile its layout can hold (the list says which are live)
        tiles = {}
        if max_q > 1:
            for tq in lay.tile_sizes:
                cap = lay.tile_cap(tq)
                total, n_multi, n_single = (cap, cap, nb if singles else 0) if all_tiles else self._tile_counts.get(tq, (0, 0, 0))
                a, m = o[f"qtiles_{tq}"], o[f"qtiles_multi_{tq}"]
                tiles[tq] = QueryTiles(dev[a : a + 2 * cap], total, dev[m : m + 2 * cap], n_multi, n_single)
        view = lambda name, size: dev[o[name] : o[name] + size]  # noqa: E731
        tables, slots = [], []
        for g in range(self.n_groups):
            tb = o["tables"] + g * lay.b_cap * lay.width
            tables.append(dev[tb : tb + nb * lay.width].view(nb, lay.width))
            sb = o["slots"] + g * lay.n_cap
            slots.append(dev[sb : sb + n])
        return StepContext(
            rt=self.rt,
            num_tokens=n,
            num_seqs=nb,
            token_ids=view("token_ids", n),
            positions=view("positions", n),
            feedback_rows=view("feedback_rows", n) if self.token_feedback is not None else None,
            token_feedback=self.token_feedback,
            query_start_loc=view("qsl", nb + 1),
            context_lens=view("ctx", nb),
            state_slots=view("state_slots", nb),
            logit_rows=view("logit_rows", max(r, 1)),
            num_logit_rows=r,
            block_tables=tables,
            slot_mappings=slots,
            max_query_len=max_q,
            max_context_len=max_ctx,
            block_size=self.block_size,
            h_query_start_loc=host[o["qsl"] : o["qsl"] + nb + 1].copy(),
            h_context_lens=host[o["ctx"] : o["ctx"] + nb].copy(),
            h_state_slots=host[o["state_slots"] : o["state_slots"] + nb].copy(),
            context_bound=bound,
            query_tiles=tiles,
        )

    # ------------------------------------------------------------------ running
    def step(self, items: Sequence[BatchItem]) -> torch.Tensor:
        """Run one batch.  Returns float logits ``[R, vocab]`` on the device, rows ordered by
        item, then by the item's wanted places.  The tensor is a view of a buffer that the
        next step overwrites."""
        if not items:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        ops.set_pdl(self.pdl)
        if self.state_slots is not None:
            fresh = self.state_slots.take_fresh()
            if fresh and self._pool is not None:
                self._pool.clear_state_slots(fresh)
        single = all(len(it.token_ids) == 1 and it.wanted() == [0] for it in items)
        if self.cuda_graphs and single and len(items) <= self.graph_buckets[-1]:
            bucket = next(b for b in self.graph_buckets if b >= len(items))
            return self._step_graph(items, bucket, bucket, decode_form=True)
        n_tok = sum(len(it.token_ids) for it in items)
        if n_tok > self.rt.max_tokens or len(items) > self.rt.max_seqs:
            raise ValueError(
                f"a step of {n_tok} tokens in {len(items)} requests exceeds the runner's limits "
                f"({self.rt.max_tokens} tokens, {self.rt.max_seqs} requests)"
            )
        n_rows = sum(len(it.wanted()) for it in items)
        if self.cuda_graphs and n_tok >= MIN_GRAPH_TOKENS and len(items) <= self.graph_buckets[-1]:
            # A step of many tokens launches some 130 kernels; replayed as a graph they follow one
            # another without the gaps of launches from Python.  Tokens are padded to a multiple of
            # GRAPH_TOKEN_STEP, sequences to a bucket; the padding belongs to no sequence.
            b_cap = next(b for b in self.graph_buckets if b >= len(items))
            n_cap = min(self.rt.max_tokens, -(-n_tok // GRAPH_TOKEN_STEP) * GRAPH_TOKEN_STEP)
            if n_rows <= b_cap and n_cap >= n_tok:
                key = self._graph_key(items, n_cap, b_cap, decode_form=False)
                seen = self._graph_seen.get(key, 0) + 1
                self._graph_seen[key] = seen
                if seen >= self.graph_after:  # a shape that comes once is not worth a capture
                    return self._step_graph(items, n_cap, b_cap, decode_form=False)
        width = max(-(-(it.start_pos + len(it.token_ids)) // self.block_size) for it in items)
        lay = self._layout(n_tok, len(items), width, n_rows)
        self._ensure(lay.total)
        n, nb, r, max_q, max_ctx = self._fill(items, lay)
        self._upload(lay.total)
        ctx = self._context(lay, n, nb, r, max_q, max_ctx, bound=0)
        before = ops.launch_count
        logits = self.model.forward(ctx)
        self.num_kernel_launches += ops.launch_count - before
        self.num_forward_passes += 1
        self.num_tokens_processed += n
        return logits[:r]

    _pool = None

    def attach_pool(self, pool) -> None:
        self._pool = pool
        self.model.attach_cache(pool.caches)

    def _graph_key(self, items: Sequence[BatchItem], n_cap: int, b_cap: int, decode_form: bool) -> tuple:
        # A graph fixes its grids, so it is made for contexts up to a bound: the next power of two
        # (kernels whose grid follows the longest context then launch at most twice what they need).
        max_ctx = max(it.start_pos + len(it.token_ids) for it in items)
        reach = min(self.max_model_len, max(MIN_GRAPH_CONTEXT, 1 << max(0, max_ctx - 1).bit_length()))
        # a step of many tokens is captured once for batches with single-token sequences among them
        # (those go to the decode kernel) and once for batches without
        singles = (not decode_form) and any(len(it.token_ids) == 1 for it in items)
        return (n_cap, b_cap, reach, singles, bool(decode_form))

    def _step_graph(self, items: Sequence[BatchItem], n_cap: int, b_cap: int, decode_form: bool) -> torch.Tensor:
        """Replay the step as a graph made for ``n_cap`` tokens in ``b_cap`` sequences.
        ``decode_form``: every sequence brings one token and wants its logits (then ``n_cap ==
        b_cap``); else a sequence may bring any number of the tokens."""
        lay = self._layout(n_cap, b_cap, self.max_width, b_cap)
        self._ensure(lay.total)
        key = self._graph_key(items, n_cap, b_cap, decode_form)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(key, lay)
        n, _, r, max_q, max_ctx = self._fill(items, lay, padded=True, tiles=not decode_form)
        self._upload(lay.total)
        graph, logits = entry
        graph.replay()
        self.num_kernel_launches += self.graph_kernels[key]
        self.num_graph_kernels += self.graph_kernels[key]
        self.num_forward_passes += 1
        self.num_tokens_processed += n
        return logits[:r]

    def _capture(self, key: tuple, lay: _Layout):
        """Make the graph of a shape.  Nothing of the step that asked for it runs here: the one
        eager run that sizes every buffer and loads every kernel outside the capture sees a batch
        of padding only (no sequence has a query, no token has a slot), so it writes no key, no
        value and no state; the step's own arrays go to the device afterwards and the step runs
        once, as the first replay."""
        n_cap, b_cap, reach, singles, decode_form = key
        self._fill((), lay, padded=True, tiles=not decode_form)
        self._upload(lay.total)
        # one token per sequence: the decode form; else a sequence may bring up to all the tokens
        ctx = self._context(lay, n_cap, b_cap, b_cap, 1 if decode_form else n_cap, reach, bound=reach, all_tiles=True, singles=singles)
        self.model.forward(ctx)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        self.rt.capturing = True
        before = ops.launch_count
        try:
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
        finally:
            self.rt.capturing = False
        self.graph_kernels[key] = ops.launch_count - before
        self.rt.graphs_captured = True
        self._graphs[key] = (graph, logits)
        return self._graphs[key]
