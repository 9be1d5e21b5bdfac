"""Serving figures: throughput, latency percentiles, cache use.  A slim form of
umarhassan-cloud/kvforge's ``MetricsCollector`` (src/tokenvault/metrics.py:40-111), without
the cost model."""

from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np


def percentile(values: list[float], q: float) -> float:
    return float(np.percentile(values, q)) if values else float("nan")


@dataclass
class MetricsCollector:
    start_time: float = field(default_factory=time.perf_counter)
    end_time: float | None = None
    num_steps: int = 0
    num_prompt_tokens: int = 0
    num_generated_tokens: int = 0
    num_finished: int = 0
    num_aborted: int = 0
    ttft: list[float] = field(default_factory=list)
    tpot: list[float] = field(default_factory=list)
    e2e: list[float] = field(default_factory=list)
    batch_sizes: list[int] = field(default_factory=list)
    batched_tokens: list[int] = field(default_factory=list)
    kv_utilization: list[float] = field(default_factory=list)
    step_times: list[float] = field(default_factory=list)

    def reset(self) -> None:
        self.__init__()  # type: ignore[misc]

    def record_step(self, batch_size: int, num_tokens: int, step_time: float, kv_utilization: float) -> None:
        self.num_steps += 1
        self.batch_sizes.append(batch_size)
        self.batched_tokens.append(num_tokens)
        self.step_times.append(step_time)
        self.kv_utilization.append(kv_utilization)

    def record_finished(self, req) -> None:
        if req.finish_reason is not None and req.finish_reason.value == "abort":
            self.num_aborted += 1
            return
        self.num_finished += 1
        self.num_prompt_tokens += req.num_prompt_tokens
        self.num_generated_tokens += req.num_output_tokens
        for value, into in ((req.ttft, self.ttft), (req.tpot, self.tpot), (req.e2e_latency, self.e2e)):
            if value is not None:
                into.append(value)

    def summary(self) -> dict[str, float]:
        end = self.end_time or time.perf_counter()
        elapsed = max(end - self.start_time, 1e-9)
        return {
            "elapsed_s": elapsed,
            "requests_finished": float(self.num_finished),
            "requests_per_s": self.num_finished / elapsed,
            "generated_tokens": float(self.num_generated_tokens),
            "output_tokens_per_s": self.num_generated_tokens / elapsed,
            "total_tokens_per_s": (self.num_generated_tokens + self.num_prompt_tokens) / elapsed,
            "ttft_p50_ms": percentile(self.ttft, 50) * 1e3,
            "ttft_p99_ms": percentile(self.ttft, 99) * 1e3,
            "tpot_p50_ms": percentile(self.tpot, 50) * 1e3,
            "tpot_p99_ms": percentile(self.tpot, 99) * 1e3,
            "e2e_p50_ms": percentile(self.e2e, 50) * 1e3,
            "e2e_p99_ms": percentile(self.e2e, 99) * 1e3,
            "mean_batch_size": float(np.mean(self.batch_sizes)) if self.batch_sizes else 0.0,
            "peak_kv_utilization": max(self.kv_utilization, default=0.0),
            "num_steps": float(self.num_steps),
        }
