"""Request state machine: WAITING -> RUNNING -> FINISHED, RUNNING -> WAITING on preemption,
any live state -> ABORTED.  Fields, properties and the stop rules are those of
umarhassan-cloud/kvforge's ``Request`` and ``RequestOutput``
(src/tokenvault/batching/request.py:22-150), without the draft-model counter and priority.
Preemption is by recomputation: pages are given back and ``num_computed_tokens`` is reset,
and on re-admission the prompt and the tokens generated so far are run again.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum

from ..sampling.params import SamplingParams


class RequestStatus(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"

    @property
    def is_final(self) -> bool:
        return self in (RequestStatus.FINISHED, RequestStatus.ABORTED)


class FinishReason(str, Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"


@dataclass(eq=False)
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    arrival_time: float = field(default_factory=time.perf_counter)
    eos_token_id: int | None = None

    status: RequestStatus = RequestStatus.WAITING
    finish_reason: FinishReason | None = None
    output_token_ids: list[int] = field(default_factory=list)
    # Tokens whose keys and values are in the cache.  While decoding:
    # num_computed_tokens == num_tokens - 1 (the newest token is the next query).
    num_computed_tokens: int = 0
    num_preemptions: int = 0
    stream_base: int = 0  # first key of the request's random stream

    first_scheduled_time: float | None = None
    first_token_time: float | None = None
    finish_time: float | None = None
    token_times: list[float] = field(default_factory=list)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_uncomputed_tokens(self) -> int:
        return self.num_tokens - self.num_computed_tokens

    @property
    def is_prefill(self) -> bool:
        """True until every token but the newest is in the cache (request.py:83-86)."""
        return self.num_output_tokens == 0 or self.num_uncomputed_tokens > 1

    @property
    def is_finished(self) -> bool:
        return self.status.is_final

    def append_token(self, token_id: int, now: float | None = None) -> None:
        now = time.perf_counter() if now is None else now
        self.output_token_ids.append(token_id)
        self.token_times.append(now)
        if self.first_token_time is None:
            self.first_token_time = now

    def check_stop(self, max_model_len: int) -> FinishReason | None:
        """request.py:99-110."""
        params = self.sampling_params
        last = self.output_token_ids[-1] if self.output_token_ids else None
        if last is not None and not params.ignore_eos and (last == self.eos_token_id or last in params.stop_token_ids):
            return FinishReason.STOP
        if self.num_output_tokens >= params.max_tokens or self.num_tokens >= max_model_len:
            return FinishReason.LENGTH
        return None

    @property
    def ttft(self) -> float | None:
        return None if self.first_token_time is None else self.first_token_time - self.arrival_time

    @property
    def e2e_latency(self) -> float | None:
        return None if self.finish_time is None else self.finish_time - self.arrival_time

    @property
    def tpot(self) -> float | None:
        if len(self.token_times) < 2:
            return None
        return (self.token_times[-1] - self.token_times[0]) / (len(self.token_times) - 1)


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list[int]
    output_token_ids: list[int]
    new_token_ids: list[int]
    finished: bool
    finish_reason: FinishReason | None = None
    text: str | None = None

    @classmethod
    def from_request(cls, req: Request, new_token_ids: list[int]) -> RequestOutput:
        return cls(
            request_id=req.request_id,
            prompt_token_ids=req.prompt_token_ids,
            output_token_ids=list(req.output_token_ids),
            new_token_ids=new_token_ids,
            finished=req.is_finished,
            finish_reason=req.finish_reason,
        )
