"""Device-side run state shared by the parts: storage type, persistent activation
buffers, the device error flag, and the step's batch description (``StepContext``)."""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


class Runtime:
    """Owns the activation buffers.  A buffer is asked for by name and width and is kept for
    the life of the runtime, so that the same addresses are used every step (a captured
    CUDA graph can be replayed) and no step allocates."""

    def __init__(self, device: str | torch.device, dtype: torch.dtype, max_tokens: int, max_seqs: int, max_model_len: int = 0, lazy: bool = False) -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("kvforge_b200 runs on a CUDA device only (there is no CPU path)")
        self.dtype = dtype
        self.max_tokens = int(max_tokens)
        self.max_seqs = int(max_seqs)
        self.max_model_len = int(max_model_len)
        # lazy: a buffer is made for the rows asked for (rounded up), not for the whole token budget
        self.lazy = bool(lazy)
        self._buffers: dict[tuple, torch.Tensor] = {}
        # One int32 per sequence for tokens sampled on the device, then the device error flag: a step's
        # tokens and the flag reach the host in one copy.
        self.status = torch.zeros(self.max_seqs + 1, dtype=torch.int32, device=self.device)
        self.sampled_tokens = self.status[: self.max_seqs]
        self.err = self.status[self.max_seqs :]
        # Tile sizes (queries of one sequence per CTA) of kernels that want a list of query tiles with
        # every step; parts add theirs in ``bind``, the step function fills ``StepContext.query_tiles``.
        self.query_tile_sizes: set[int] = set()
        self.capturing = False
        self.graphs_captured = False  # captured graphs hold buffer addresses: no buffer may move afterwards
        self._side: torch.cuda.Stream | None = None

    def side_stream(self) -> torch.cuda.Stream:
        """A second stream for a kernel that may run beside the step's chain while a step is captured
        (a branch of the graph); whoever uses it makes the step's stream wait for it again."""
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    def buf(self, name: str, rows: int, cols: int, dtype: torch.dtype | None = None, cap: int | None = None) -> torch.Tensor:
        """A ``[rows, cols]`` view of the persistent buffer ``name`` (contents undefined).
        It is made for ``cap`` rows (default: the token budget of a step) and grows if more
        are asked for."""
        dtype = dtype or self.dtype
        key = (name, cols, dtype)
        t = self._buffers.get(key)
        if t is None or t.shape[0] < rows:
            if self.capturing or (self.graphs_captured and t is not None):
                raise RuntimeError(f"buffer {name} would have to grow after or during graph capture")
            if self.lazy:
                cap = 1 << max(4, (max(rows, 1) - 1).bit_length())
            else:
                cap = max(rows, self.max_tokens if cap is None else cap)
            t = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._buffers[key] = t
        return t[:rows]

    def check_error_flag(self) -> None:
        flag = int(self.err.item())
        if flag:
            self.err.zero_()
            what = []
            if flag & 1:
                what.append("a token id outside the vocabulary")
            if flag & 2:
                what.append("a cache slot outside the pool")
            if flag & 4:
                what.append("a bounded wait inside a kernel ran out")
            raise RuntimeError("device-side check failed: " + ", ".join(what or [f"flag {flag}"]))


@dataclass
class QueryTiles:
    """A step's tiles of queries for kernels that take ``size`` queries of one sequence per CTA:
    int32 pairs (sequence or -1, first query of the tile), the longest walk over the keys first."""

    tiles: torch.Tensor  # of all sequences
    count: int  # how many of them to launch
    multi: torch.Tensor  # of the sequences that bring more than one query
    multi_count: int
    num_single: int  # sequences that bring exactly one query (a captured step: as many as it has sequences)


@dataclass
class StepContext:
    """One step's batch as the parts see it.  All device arrays are int32."""

    rt: Runtime
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # [N]
    positions: torch.Tensor  # [N] absolute position of each token
    query_start_loc: torch.Tensor  # [B+1]
    context_lens: torch.Tensor  # [B] tokens in the cache after this step's writes
    state_slots: torch.Tensor  # [B] slot of each request's fixed-size state
    logit_rows: torch.Tensor  # [R] flat token rows whose logits are wanted
    num_logit_rows: int
    block_tables: list[torch.Tensor]  # per cache group: [B, W]
    slot_mappings: list[torch.Tensor]  # per cache group: [N]
    max_query_len: int
    max_context_len: int
    block_size: int
    # Host copies, for parts that walk sequences on the host (test parts do).
    h_query_start_loc: np.ndarray | None = None
    h_context_lens: np.ndarray | None = None
    h_state_slots: np.ndarray | None = None
    # Where a token comes from the device: per token a row of ``token_feedback`` or -1.
    feedback_rows: torch.Tensor | None = None
    token_feedback: torch.Tensor | None = None
    # The step's float residual stream [N, hidden], set by the model before its blocks run.  A mixer
    # or feed-forward may add its result into it directly and return ``ops.ADDED`` instead of a tensor.
    residual: torch.Tensor | None = None
    # Upper bound on any context (fixes grid sizes of captured decode steps).
    context_bound: int = 0
    # Per registered tile size a ``QueryTiles``.  Empty when every sequence brings one token.
    query_tiles: dict = field(default_factory=dict)
    extras: dict = field(default_factory=dict)

    @property
    def all_single_query(self) -> bool:
        return self.max_query_len == 1
