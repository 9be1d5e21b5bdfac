"""A request's life in this engine, and what a caller gets back from it.

States and reasons carry the names of umarhassan-cloud/kvforge
(src/tokenvault/batching/request.py:22-36: waiting, running, finished, aborted; stop, length,
abort), and so do the counters the scheduler steers by (``num_computed_tokens``, ``is_prefill``:
request.py:51-53,83-86).  The life cycle itself is this engine's own:

* A sampled token is first *launched*: the kernel that draws it has been queued, its value is
  still on the device.  The request reserves its place in the output (``launch_token``), which
  makes it schedulable for the next step at once; that step's embedding lookup takes the token
  from the device.
* One step later the value is read and *landed* (``land_token``): it replaces the placeholder,
  gets its time stamp (the moment the token exists for a caller, which is what the latency
  figures mean), and is checked against the stop tokens.
* A stop by count (``max_tokens``, the model's length) needs no value and is known at launch.
* Preemption is by recomputation: the pages go back, ``num_computed_tokens`` returns to zero and
  the prompt and the tokens generated so far run again.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from enum import Enum

import numpy as np

from ..sampling.params import SamplingParams

IN_FLIGHT = -1  # stands in an output list for a token whose value is still on the device


class RequestStatus(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


class FinishReason(str, Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"


_FINAL = (RequestStatus.FINISHED, RequestStatus.ABORTED)


class Request:
    __slots__ = (
        "request_id", "prompt_token_ids", "sampling_params", "arrival_time", "eos_token_id", "stream_base",
        "status", "finish_reason", "output_token_ids", "num_computed_tokens", "num_preemptions",
        "first_scheduled_time", "finish_time", "token_times", "_prompt_array",
    )  # fmt: skip

    def __init__(
        self,
        request_id: str,
        prompt_token_ids: list[int],
        sampling_params: SamplingParams | None = None,
        arrival_time: float | None = None,
        eos_token_id: int | None = None,
        stream_base: int = 0,
    ) -> None:
        self.request_id = request_id
        self.prompt_token_ids = prompt_token_ids
        self.sampling_params = sampling_params if sampling_params is not None else SamplingParams()
        self.arrival_time = time.perf_counter() if arrival_time is None else arrival_time
        self.eos_token_id = eos_token_id
        self.stream_base = stream_base  # first key of the request's random stream
        self.status = RequestStatus.WAITING
        self.finish_reason: FinishReason | None = None
        self.output_token_ids: list[int] = []
        # Tokens whose keys and values are in the cache.  While decoding this is num_tokens - 1:
        # the newest token is the next query.
        self.num_computed_tokens = 0
        self.num_preemptions = 0
        self.first_scheduled_time: float | None = None
        self.finish_time: float | None = None
        self.token_times: list[float | None] = []  # per output token: when its value reached the host
        self._prompt_array = None  # the prompt as an int32 array, made when a portion of it is first asked for

    def __repr__(self) -> str:
        return f"Request({self.request_id!r}, {self.status.value}, {self.num_computed_tokens}/{self.num_tokens} tokens)"

    # ------------------------------------------------------------------ counts
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
        """Whether more than the newest token is missing from the cache: before the first
        sampled token, and again after a preemption."""
        return not self.output_token_ids or self.num_uncomputed_tokens > 1

    @property
    def is_finished(self) -> bool:
        return self.status in _FINAL

    def tokens(self, start: int, count: int):
        """``count`` known tokens from position ``start`` (prompt, then output): a list, or for a
        portion that lies inside the prompt a slice of an int32 array of it (a step copies
        thousands of prompt tokens into its arrays; from a list that is a conversion per token)."""
        n_prompt = len(self.prompt_token_ids)
        end = start + count
        if end <= n_prompt:
            if count < 64:
                return self.prompt_token_ids[start:end]
            if self._prompt_array is None:
                self._prompt_array = np.asarray(self.prompt_token_ids, dtype=np.int32)
            return self._prompt_array[start:end]
        if start >= n_prompt:
            return self.output_token_ids[start - n_prompt : end - n_prompt]
        return self.prompt_token_ids[start:] + self.output_token_ids[: end - n_prompt]

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    # ------------------------------------------------------------------ tokens on their way
    @property
    def has_token_in_flight(self) -> bool:
        return bool(self.output_token_ids) and self.output_token_ids[-1] == IN_FLIGHT

    def in_flight_within(self, start: int) -> bool:
        """Whether any token from position ``start`` on is still on the device."""
        first = max(0, start - len(self.prompt_token_ids))
        return IN_FLIGHT in self.output_token_ids[first:]

    def launch_token(self) -> int:
        """Reserve the place of a token that a queued kernel will sample; returns its index in
        the output."""
        self.output_token_ids.append(IN_FLIGHT)
        self.token_times.append(None)
        return len(self.output_token_ids) - 1

    def land_token(self, index: int, token_id: int, now: float | None = None) -> None:
        """The value of output token ``index`` has reached the host."""
        self.output_token_ids[index] = token_id
        self.token_times[index] = time.perf_counter() if now is None else now

    def append_token(self, token_id: int, now: float | None = None) -> None:
        """Launch and land in one go (a token whose value is known at once)."""
        self.land_token(self.launch_token(), token_id, now)

    def truncate_output(self, length: int) -> None:
        """Drop every output token from ``length`` on (what was launched after a stop token)."""
        del self.output_token_ids[length:]
        del self.token_times[length:]

    def drop_token_in_flight(self) -> None:
        if self.has_token_in_flight:
            self.truncate_output(len(self.output_token_ids) - 1)

    # ------------------------------------------------------------------ stops
    def stops_at(self, token_id: int) -> bool:
        """Whether this token ends the request (request.py:99-105: the end-of-sequence token or
        one of ``stop_token_ids``, unless ``ignore_eos``)."""
        p = self.sampling_params
        if p.ignore_eos:
            return False
        return token_id == self.eos_token_id or token_id in p.stop_token_ids

    def at_count_limit(self, max_model_len: int) -> bool:
        """Whether the request has as many tokens as it may have (request.py:106-109); true
        whatever the value of its newest token."""
        return self.num_output_tokens >= self.sampling_params.max_tokens or self.num_tokens >= max_model_len

    # ------------------------------------------------------------------ latencies
    def _landed_times(self) -> list[float]:
        return [t for t in self.token_times if t is not None]

    @property
    def first_token_time(self) -> float | None:
        times = self._landed_times()
        return times[0] if times else None

    @property
    def ttft(self) -> float | None:
        """Arrival to first token on the host."""
        first = self.first_token_time
        return None if first is None else first - self.arrival_time

    @property
    def tpot(self) -> float | None:
        """Mean time between output tokens after the first."""
        times = self._landed_times()
        if len(times) < 2:
            return None
        return (times[-1] - times[0]) / (len(times) - 1)

    @property
    def e2e_latency(self) -> float | None:
        return None if self.finish_time is None else self.finish_time - self.arrival_time


@dataclass
class RequestOutput:
    """What ``InferenceEngine.step`` reports for a request that got a token
    (request.py:130-139)."""

    request_id: str
    prompt_token_ids: list[int]
    output_token_ids: list[int]
    new_token_ids: list[int]
    finished: bool
    finish_reason: FinishReason | None = None
    text: str | None = None
