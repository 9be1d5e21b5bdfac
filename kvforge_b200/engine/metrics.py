"""Serving figures of an engine: how many tokens and requests per second, how long a caller
waited for the first token and between tokens, how full the steps and the cache were.

The figures and the names they are reported under are those of umarhassan-cloud/kvforge's
collector (src/tokenvault/metrics.py:40-111) without its cost model.  Latencies are taken from the
times at which token values reached the host (``Request.token_times``), so with tokens read a step
late they are what a caller of ``step()`` sees, not when a kernel was queued.
"""

from __future__ import annotations

import math
import time


class _Samples:
    """A growing list of observations with the few statistics the summary needs."""

    def __init__(self) -> None:
        self.values: list[float] = []

    def add(self, value: float | None) -> None:
        if value is not None:
            self.values.append(float(value))

    def quantile_ms(self, q: float) -> float:
        """The ``q``-th percentile (linear between neighbours) in milliseconds; NaN without data."""
        v = sorted(self.values)
        if not v:
            return math.nan
        at = (len(v) - 1) * q / 100.0
        lo = int(at)
        hi = min(lo + 1, len(v) - 1)
        return 1e3 * (v[lo] + (v[hi] - v[lo]) * (at - lo))

    def mean(self) -> float:
        return sum(self.values) / len(self.values) if self.values else 0.0

    def peak(self) -> float:
        return max(self.values, default=0.0)


class MetricsCollector:
    def __init__(self) -> None:
        self.reset()

    def reset(self) -> None:
        self.start_time = time.perf_counter()
        self.end_time: float | None = None
        self.num_steps = 0
        self.num_finished = 0
        self.num_aborted = 0
        self.num_prompt_tokens = 0
        self.num_generated_tokens = 0
        self.ttft, self.tpot, self.e2e = _Samples(), _Samples(), _Samples()
        self.batch_sizes, self.batched_tokens = _Samples(), _Samples()
        self.step_times, self.kv_utilization = _Samples(), _Samples()

    def record_step(self, batch_size: int, num_tokens: int, step_time: float, kv_utilization: float) -> None:
        self.num_steps += 1
        self.batch_sizes.add(batch_size)
        self.batched_tokens.add(num_tokens)
        self.step_times.add(step_time)
        self.kv_utilization.add(kv_utilization)

    def record_finished(self, req) -> None:
        """A request has ended; an aborted one counts as such and adds no tokens or latencies."""
        if req.finish_reason is not None and req.finish_reason.value == "abort":
            self.num_aborted += 1
            return
        self.num_finished += 1
        self.num_prompt_tokens += req.num_prompt_tokens
        self.num_generated_tokens += req.num_output_tokens
        self.ttft.add(req.ttft)
        self.tpot.add(req.tpot)
        self.e2e.add(req.e2e_latency)

    def summary(self) -> dict[str, float]:
        elapsed = max((self.end_time or time.perf_counter()) - self.start_time, 1e-9)
        out = {
            "elapsed_s": elapsed,
            "requests_finished": float(self.num_finished),
            "requests_aborted": float(self.num_aborted),
            "requests_per_s": self.num_finished / elapsed,
            "generated_tokens": float(self.num_generated_tokens),
            "output_tokens_per_s": self.num_generated_tokens / elapsed,
            "total_tokens_per_s": (self.num_generated_tokens + self.num_prompt_tokens) / elapsed,
        }
        for name, samples in (("ttft", self.ttft), ("tpot", self.tpot), ("e2e", self.e2e)):
            for q in (50, 99):
                out[f"{name}_p{q}_ms"] = samples.quantile_ms(q)
        out["mean_batch_size"] = self.batch_sizes.mean()
        out["mean_batched_tokens"] = self.batched_tokens.mean()
        out["mean_step_ms"] = 1e3 * self.step_times.mean()
        out["peak_kv_utilization"] = self.kv_utilization.peak()
        out["num_steps"] = float(self.num_steps)
        return out
