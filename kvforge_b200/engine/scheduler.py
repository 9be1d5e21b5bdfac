"""Which requests run in the next step, and with how many tokens each.

The policy is that of umarhassan-cloud/kvforge's scheduler (src/tokenvault/scheduler.py:160-224),
first come first served at the level of single steps:

* Requests that already run are served before anybody new, oldest arrival first.  One that is
  decoding takes a single token; one that still has known tokens outside the cache (a prompt, or
  prompt plus generated tokens after a preemption) takes as many as the step's token budget has
  left, so a long prompt is cut into portions that share steps with decoding requests.
* If the pages for a request's next tokens cannot be had, the latest arrival among the running
  requests that have not been served yet in this pass gives way: its pages and its state slot go
  back, it waits again (at its old place in the order of arrival) and will be recomputed.  With
  nobody left to evict, the request itself gives way.
* A pass that evicted somebody admits nobody.  Otherwise waiting requests are admitted strictly in
  order of arrival, and the first that does not fit (tokens, ``max_num_seqs``, pages above the
  watermark, a free state slot) ends the admission: nobody overtakes it.

``max_prefill_chunk`` (not in kvforge) caps one request's portion in a step.
"""

from __future__ import annotations

import bisect
import itertools
import time
from dataclasses import dataclass, field

from ..cache.block_manager import BlockManager
from ..cache.state_slots import StateSlotPool
from ..config.engine_config import SchedulerConfig
from .request import FinishReason, Request, RequestStatus


class RequestRejectedError(ValueError):
    """The request can never be served by this engine as configured."""


@dataclass
class ScheduledRequest:
    request: Request
    num_new_tokens: int
    is_prefill: bool


@dataclass
class SchedulerOutput:
    """One pass's decisions: who runs (in the order of the batch) and who was evicted."""

    scheduled: list[ScheduledRequest] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)

    @property
    def is_empty(self) -> bool:
        return len(self.scheduled) == 0

    @property
    def num_batched_tokens(self) -> int:
        return sum(s.num_new_tokens for s in self.scheduled)

    @property
    def prefills(self) -> list[ScheduledRequest]:
        return [s for s in self.scheduled if s.is_prefill]

    @property
    def decodes(self) -> list[ScheduledRequest]:
        return [s for s in self.scheduled if not s.is_prefill]


class Scheduler:
    def __init__(self, config: SchedulerConfig, block_manager: BlockManager, state_slots: StateSlotPool | None = None) -> None:
        self.config = config
        self.block_manager = block_manager
        self.state_slots = state_slots
        self.requests: dict[str, Request] = {}  # every live request, waiting or running
        self.running: list[Request] = []
        # waiting requests sorted by (arrival, order of submission); a preempted request comes back
        # with its old arrival time and so to the front of later arrivals
        self._waiting: list[tuple[float, int, Request]] = []
        self._ticket = itertools.count()
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queues
    @property
    def num_waiting(self) -> int:
        return len(self._waiting)

    @property
    def num_running(self) -> int:
        return len(self.running)

    def has_unfinished(self) -> bool:
        return bool(self.running or self._waiting)

    def _enqueue(self, req: Request) -> None:
        req.status = RequestStatus.WAITING
        bisect.insort(self._waiting, (req.arrival_time, next(self._ticket), req), key=lambda e: e[:2])

    def _dequeue(self, req: Request) -> None:
        self._waiting = [e for e in self._waiting if e[2] is not req]

    def _give_back(self, req: Request) -> None:
        """Pages and state slot of a request that stops running (for good or for now)."""
        self.block_manager.free(req.request_id)
        if self.state_slots is not None:
            self.state_slots.free(req.request_id)

    # ------------------------------------------------------------------ arrivals and departures
    def add_request(self, req: Request) -> None:
        """Refuses what could never run (scheduler.py:109-129): a second request of the same name,
        an empty prompt, a prompt that leaves no room under ``max_model_len``, a prompt above the
        token budget when it may not be cut, and a request whose pages the pool can never hold."""
        cfg = self.config
        n_prompt = req.num_prompt_tokens
        if req.request_id in self.requests:
            raise RequestRejectedError(f"a request named {req.request_id!r} is already live")
        if n_prompt == 0:
            raise RequestRejectedError("the prompt is empty")
        if n_prompt >= cfg.max_model_len:
            raise RequestRejectedError(f"a prompt of {n_prompt} tokens leaves no room under max_model_len = {cfg.max_model_len}")
        if not cfg.enable_chunked_prefill and n_prompt > cfg.max_num_batched_tokens:
            raise RequestRejectedError(f"a prompt of {n_prompt} tokens exceeds max_num_batched_tokens = {cfg.max_num_batched_tokens} and prompts are not cut")
        longest = min(n_prompt + req.sampling_params.max_tokens, cfg.max_model_len)
        largest_portion = self._portion(longest, cfg.max_num_batched_tokens) if cfg.enable_chunked_prefill else longest
        if not self.block_manager.can_ever_fit(longest, largest_portion):
            raise RequestRejectedError(f"{longest} tokens can never fit the pages of the cache")
        self.requests[req.request_id] = req
        self._enqueue(req)

    def finish_request(self, req: Request, reason: FinishReason) -> None:
        """Ends a request for good and gives back what it holds."""
        was_waiting = req.status == RequestStatus.WAITING
        req.finish_reason = reason
        req.status = RequestStatus.ABORTED if reason is FinishReason.ABORT else RequestStatus.FINISHED
        req.finish_time = time.perf_counter()
        if was_waiting:
            self._dequeue(req)
        else:
            self.running = [r for r in self.running if r is not req]
        self._give_back(req)
        self.requests.pop(req.request_id, None)

    def abort_request(self, request_id: str) -> Request | None:
        req = self.requests.get(request_id)
        if req is None or req.is_finished:
            return None
        self.finish_request(req, FinishReason.ABORT)
        return req

    def _evict(self, req: Request, plan: SchedulerOutput) -> None:
        self._give_back(req)
        req.num_computed_tokens = 0
        req.num_preemptions += 1
        self.num_preemptions += 1
        self._enqueue(req)
        plan.preempted.append(req)

    # ------------------------------------------------------------------ one pass
    def _portion(self, missing: int, budget: int) -> int:
        """How many of a request's ``missing`` tokens one step takes."""
        cfg = self.config
        if not cfg.enable_chunked_prefill:
            return missing
        cap = cfg.max_prefill_chunk or missing
        return min(missing, budget, cap)

    def schedule(self) -> SchedulerOutput:
        plan = SchedulerOutput()
        budget = self._serve_running(plan, self.config.max_num_batched_tokens)
        if not plan.preempted:
            self._admit_waiting(plan, budget)
        return plan

    def _serve_running(self, plan: SchedulerOutput, budget: int) -> int:
        """Running requests, oldest first; evictions come from the young end of the same order.
        Returns what is left of the token budget."""
        bm = self.block_manager
        order = sorted(self.running, key=lambda r: r.arrival_time)
        first, end = 0, len(order)  # order[first:end] have not been decided yet
        kept: list[Request] = []
        while first < end:
            req = order[first]
            first += 1
            have = req.num_computed_tokens
            take = self._portion(req.num_uncomputed_tokens, budget) if req.is_prefill else req.num_uncomputed_tokens
            if take < 1 or take > budget:
                kept.append(req)  # no room for it in this step; it keeps its pages
                continue
            while not bm.can_append_slots(req.request_id, have + take, have) and first < end:
                end -= 1
                self._evict(order[end], plan)
            if not bm.can_append_slots(req.request_id, have + take, have):
                self._evict(req, plan)  # nobody younger is left to make room
                continue
            bm.append_slots(req.request_id, have + take, have)
            plan.scheduled.append(ScheduledRequest(req, take, req.is_prefill))
            kept.append(req)
            budget -= take
        self.running = kept
        return budget

    def _admit_waiting(self, plan: SchedulerOutput, budget: int) -> None:
        cfg, bm, slots = self.config, self.block_manager, self.state_slots
        now = time.perf_counter()
        while self._waiting and budget > 0 and len(self.running) < cfg.max_num_seqs:
            req = self._waiting[0][2]
            known = req.num_tokens  # after a preemption: the prompt and what was generated
            take = self._portion(known, budget)
            if take > budget:  # prompts are not cut and this one does not fit the rest of the step
                return
            if not bm.can_allocate(known, take) or (slots is not None and slots.num_free == 0):
                return  # the head of the line waits, and everybody behind it
            self._waiting.pop(0)
            req.num_computed_tokens = bm.allocate(req.request_id, known, take)
            if slots is not None:
                slots.allocate(req.request_id)
            req.status = RequestStatus.RUNNING
            if req.first_scheduled_time is None:
                req.first_scheduled_time = now
            self.running.append(req)
            plan.scheduled.append(ScheduledRequest(req, take, True))
            budget -= take
