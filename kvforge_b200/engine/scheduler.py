"""Iteration-level scheduler over the paged cache.

Policy of umarhassan-cloud/kvforge's ``Scheduler`` (src/tokenvault/scheduler.py:68-224), first
come first served:

1. Running requests first, in arrival order: a decoding request takes one token, a request
   still in its prompt takes ``min(rest, budget)`` tokens (chunked prefill).
2. When pages run out for a running request, the *latest arrival* still waiting for its turn
   in this pass is preempted by recomputation (its pages and state slot are given back, it
   goes back to the waiting queue with its arrival time, and will run prompt plus generated
   tokens again); if nobody is left to evict, the request itself is preempted.
3. New requests are admitted only in a step that preempted nobody, head of line first
   with no skipping, while the token budget, ``max_num_seqs``, the pages (with the watermark)
   and a free state slot allow.

Added to that policy: ``max_prefill_chunk`` caps one request's portion in a step.
"""

from __future__ import annotations

import heapq
import itertools
import time
from dataclasses import dataclass, field

from ..cache.block_manager import BlockManager
from ..cache.state_slots import StateSlotPool
from ..config.engine_config import SchedulerConfig
from .request import FinishReason, Request, RequestStatus


@dataclass
class ScheduledRequest:
    request: Request
    num_new_tokens: int
    is_prefill: bool


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)

    @property
    def is_empty(self) -> bool:
        return not self.scheduled

    @property
    def num_batched_tokens(self) -> int:
        return sum(s.num_new_tokens for s in self.scheduled)

    @property
    def prefills(self) -> list[ScheduledRequest]:
        return [s for s in self.scheduled if s.is_prefill]

    @property
    def decodes(self) -> list[ScheduledRequest]:
        return [s for s in self.scheduled if not s.is_prefill]


class RequestRejectedError(ValueError):
    pass


class Scheduler:
    def __init__(self, config: SchedulerConfig, block_manager: BlockManager, state_slots: StateSlotPool | None = None) -> None:
        self.config = config
        self.block_manager = block_manager
        self.state_slots = state_slots
        self._waiting: list[tuple[tuple, Request]] = []
        self._counter = itertools.count()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self.num_preemptions = 0

    # ------------------------------------------------------------------ bookkeeping
    def _push_waiting(self, req: Request) -> None:
        heapq.heappush(self._waiting, ((req.arrival_time, next(self._counter)), req))

    def _peek_waiting(self) -> Request | None:
        while self._waiting and self._waiting[0][1].status != RequestStatus.WAITING:
            heapq.heappop(self._waiting)  # aborted entries are dropped when they surface
        return self._waiting[0][1] if self._waiting else None

    @property
    def num_waiting(self) -> int:
        return sum(1 for _, r in self._waiting if r.status == RequestStatus.WAITING)

    @property
    def num_running(self) -> int:
        return len(self.running)

    def has_unfinished(self) -> bool:
        return bool(self.running) or self._peek_waiting() is not None

    def add_request(self, req: Request) -> None:
        """Checks of scheduler.py:109-129."""
        cfg, bm = self.config, self.block_manager
        if req.request_id in self.requests:
            raise RequestRejectedError(f"duplicate request id {req.request_id}")
        if req.num_prompt_tokens == 0:
            raise RequestRejectedError("empty prompt")
        if req.num_prompt_tokens >= cfg.max_model_len:
            raise RequestRejectedError(f"prompt of {req.num_prompt_tokens} tokens exceeds max_model_len {cfg.max_model_len}")
        if not cfg.enable_chunked_prefill and req.num_prompt_tokens > cfg.max_num_batched_tokens:
            raise RequestRejectedError("prompt exceeds max_num_batched_tokens without chunked prefill")
        worst_case = min(req.num_prompt_tokens + req.sampling_params.max_tokens, cfg.max_model_len)
        portion = min(cfg.max_num_batched_tokens, cfg.max_prefill_chunk or cfg.max_num_batched_tokens)
        if not bm.can_ever_fit(worst_case, portion if cfg.enable_chunked_prefill else worst_case):
            raise RequestRejectedError("request can never fit in the KV cache")
        req.status = RequestStatus.WAITING
        self.requests[req.request_id] = req
        self._push_waiting(req)

    def _release(self, req: Request) -> None:
        self.block_manager.free(req.request_id)
        if self.state_slots is not None:
            self.state_slots.free(req.request_id)

    def _preempt(self, req: Request) -> None:
        self._release(req)
        req.status = RequestStatus.WAITING
        req.num_computed_tokens = 0
        req.num_preemptions += 1
        self.num_preemptions += 1
        self._push_waiting(req)

    def finish_request(self, req: Request, reason: FinishReason) -> None:
        req.status = RequestStatus.ABORTED if reason == FinishReason.ABORT else RequestStatus.FINISHED
        req.finish_reason = reason
        req.finish_time = time.perf_counter()
        if req in self.running:
            self.running.remove(req)
        self._release(req)
        self.requests.pop(req.request_id, None)

    def abort_request(self, request_id: str) -> Request | None:
        req = self.requests.get(request_id)
        if req is None or req.is_finished:
            return None
        self.finish_request(req, FinishReason.ABORT)
        return req

    def _chunk(self, n_new: int, budget: int) -> int:
        cfg = self.config
        if cfg.enable_chunked_prefill:
            n_new = min(n_new, budget)
            if cfg.max_prefill_chunk:
                n_new = min(n_new, cfg.max_prefill_chunk)
        return n_new

    # ------------------------------------------------------------------ schedule
    def schedule(self) -> SchedulerOutput:
        cfg, bm = self.config, self.block_manager
        out = SchedulerOutput()
        budget = cfg.max_num_batched_tokens

        queue = sorted(self.running, key=lambda r: r.arrival_time)
        still_running: list[Request] = []
        while queue:
            req = queue.pop(0)
            prefill = req.is_prefill
            n_new = req.num_uncomputed_tokens
            if prefill:
                n_new = self._chunk(n_new, budget)
            if n_new <= 0 or n_new > budget:
                still_running.append(req)
                continue
            total = req.num_computed_tokens + n_new
            fits = True
            while not bm.can_append_slots(req.request_id, total, req.num_computed_tokens):
                if not queue:
                    fits = False
                    break
                victim = queue.pop()  # latest arrival
                self._preempt(victim)
                out.preempted.append(victim)
            if not fits:
                self._preempt(req)
                out.preempted.append(req)
                continue
            bm.append_slots(req.request_id, total, req.num_computed_tokens)
            out.scheduled.append(ScheduledRequest(req, n_new, prefill))
            still_running.append(req)
            budget -= n_new
        self.running = still_running

        if out.preempted:
            return out  # no admission in a step that preempted (scheduler.py:198-199)

        now = time.perf_counter()
        while budget > 0 and len(self.running) < cfg.max_num_seqs:
            req = self._peek_waiting()
            if req is None:
                break
            n_tokens = req.num_tokens
            if not cfg.enable_chunked_prefill and n_tokens > budget:
                break
            n_new = self._chunk(n_tokens, budget)
            if not bm.can_allocate(n_tokens, n_new):
                break
            if self.state_slots is not None and self.state_slots.num_free == 0:
                break
            heapq.heappop(self._waiting)
            req.num_computed_tokens = bm.allocate(req.request_id, n_tokens, n_new)
            if self.state_slots is not None:
                self.state_slots.allocate(req.request_id)
            req.status = RequestStatus.RUNNING
            if req.first_scheduled_time is None:
                req.first_scheduled_time = now
            out.scheduled.append(ScheduledRequest(req, n_new, True))
            self.running.append(req)
            budget -= n_new
        return out
