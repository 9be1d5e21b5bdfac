"""``InferenceEngine``: the Python entry point.  One ``step()`` is one scheduler decision,
one flat forward over everything scheduled, one sampling call, and the bookkeeping.

Names and meanings follow umarhassan-cloud/kvforge's ``InferenceEngine``
(src/tokenvault/engine.py:39-297): ``add_request``, ``abort_request``,
``has_unfinished_requests``, ``generate`` (outputs in prompt order), ``step``, ``stats``.
The model is given as a folder (``config.json`` + safetensors), or is made with random
weights from ``config.model`` and ``config.seed`` as kvforge does when it is given none
(engine.py:52-54).  ``tokenizer``: for string prompts, any object with ``encode(text)``,
``decode(ids)`` and ``eos_token_id`` (``engine/tokenizer.py`` has one that needs no files).
"""

from __future__ import annotations

import itertools
import time
from collections.abc import Sequence
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, request_stream_base
from .core import EngineCore, spec_from_config, spec_from_model_dir
from .metrics import MetricsCollector
from .request import FinishReason, Request, RequestOutput
from .scheduler import ScheduledRequest, Scheduler
from .step import BatchItem


@dataclass
class _Pending:
    """A launched step whose tokens the host has not read yet."""

    sampled: list  # requests that get a token from this step, in row order
    indices: list[int]  # where in each request's output list the token goes
    host: torch.Tensor  # pinned: [rows] tokens, then the device error flag
    event: torch.cuda.Event
    rows: dict  # request id -> row
    skip: set = field(default_factory=set)  # requests that ended meanwhile


class InferenceEngine:
    def __init__(
        self,
        config: EngineConfig | None = None,
        model: str | Path | None = None,
        tokenizer: Any = None,
        init_std: float = 0.02,
    ) -> None:
        self.config = config = config or EngineConfig()
        self.tokenizer = tokenizer
        if model is not None:
            model_cfg, spec = spec_from_model_dir(model)
            config.model = model_cfg
        else:
            if config.model is None:
                raise ValueError("give a model folder or EngineConfig.model")
            spec = spec_from_config(config.model)
        config.finalize()
        self.model_config = config.model
        sc = config.scheduler
        self.core = EngineCore(
            spec,
            dtype=config.dtype,
            device=config.device,
            model_dir=model,
            seed=config.seed,
            init_std=init_std,
            cache=config.cache,
            max_num_seqs=sc.max_num_seqs,
            max_num_batched_tokens=sc.max_num_batched_tokens,
            max_model_len=sc.max_model_len,
            cuda_graphs=config.cuda_graphs,
        )
        self.block_manager = self.core.block_manager
        self.kv_cache = self.core.pool
        self.runner = self.core.runner
        self.sampler = Sampler(self.core.device, sc.max_num_seqs, tokens=self.core.rt.sampled_tokens)
        self.runner.token_feedback = self.sampler._tokens  # a sampled token can feed the next step on the device
        self._host_tokens = [torch.zeros(sc.max_num_seqs + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._flip = 0
        self._pending: _Pending | None = None
        self.scheduler = Scheduler(sc, self.block_manager, self.core.state_slots)
        self.metrics = MetricsCollector()
        self._ids = itertools.count()
        self.vocab_size = spec.vocab_size

    # ------------------------------------------------------------------ API
    def _token_ids(self, prompt: str | Sequence[int]) -> list[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a prompt given as text needs a tokenizer; give token ids or pass tokenizer=")
            ids = list(self.tokenizer.encode(prompt))
        else:
            ids = [int(t) for t in prompt]
        bad = next((t for t in ids if not 0 <= t < self.vocab_size), None)
        if bad is not None:
            raise ValueError(f"token id {bad} is outside the model's vocabulary of {self.vocab_size}")
        return ids

    def add_request(
        self,
        prompt: str | Sequence[int],
        sampling_params: SamplingParams | None = None,
        request_id: str | None = None,
        arrival_time: float | None = None,
    ) -> str:
        """Queue a prompt (text or token ids) and return the request's name (engine.py:106-134).
        The scheduler refuses what can never run (``RequestRejectedError``)."""
        ids = self._token_ids(prompt)
        name = request_id if request_id else f"req-{next(self._ids)}"
        params = sampling_params if sampling_params is not None else SamplingParams()
        eos = getattr(self.tokenizer, "eos_token_id", None) if self.tokenizer is not None else self.core.spec.eos_token_id
        self.scheduler.add_request(
            Request(name, ids, params, arrival_time, eos, stream_base=request_stream_base(self.config.seed, name, params))
        )
        return name

    def abort_request(self, request_id: str) -> bool:
        """End a live request now; whatever of it is still on the device is discarded."""
        req = self.scheduler.abort_request(request_id)
        if req is None:
            return False
        if self._pending is not None:
            self._pending.skip.add(request_id)
        req.drop_token_in_flight()
        self.metrics.record_finished(req)
        return True

    def generate(
        self,
        prompts: Sequence[str | Sequence[int]],
        sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
    ) -> list[RequestOutput]:
        """Run all prompts to their end; one output per prompt, in the order given
        (engine.py:145-159).  ``sampling_params``: one for all, or one per prompt."""
        if isinstance(sampling_params, SamplingParams) or sampling_params is None:
            per_prompt = [sampling_params] * len(prompts)
        else:
            per_prompt = list(sampling_params)
            if len(per_prompt) != len(prompts):
                raise ValueError(f"{len(per_prompt)} sampling parameter sets for {len(prompts)} prompts")
        names = [self.add_request(prompt, sp) for prompt, sp in zip(prompts, per_prompt)]
        final: dict[str, RequestOutput] = {}
        while self.has_unfinished_requests():
            final.update((out.request_id, out) for out in self.step() if out.finished)
        return [final[name] for name in names if name in final]

    # ------------------------------------------------------------------ step
    def has_unfinished_requests(self) -> bool:
        if self.scheduler.has_unfinished():
            return True
        # a launched step whose tokens have not been reported yet
        return self._pending is not None and any(r.request_id not in self._pending.skip for r in self._pending.sampled)

    def step(self) -> list[RequestOutput]:
        """One scheduler decision and one forward.  With ``async_output`` (the default) the
        tokens of a step are read from the device while the *next* step runs: a decoded token
        goes round on the device (the sampling kernel's output feeds the next embedding
        lookup), the host appends a placeholder, and patches it, checks stop tokens and
        reports the outputs one call later.  Stops by count (``max_tokens``, the model's
        length) are decided at once; a stop token is seen one step late, and the one token
        computed in between is dropped."""
        t0 = time.perf_counter()
        sched = self.scheduler.schedule()
        if sched.is_empty:
            return self._resolve(self._take_pending())
        outputs: list[RequestOutput] = []
        if self._pending is not None and any(self._needs_host_tokens(s) for s in sched.scheduled):
            # a portion of known tokens (a re-run after preemption) includes a token not read yet
            outputs += self._resolve(self._take_pending())
        previous = self._take_pending()
        self._pending = self._launch(sched.scheduled, previous)
        outputs += self._resolve(previous)
        if not self.config.async_output:
            outputs += self._resolve(self._take_pending())
        self.metrics.record_step(len(sched.scheduled), sched.num_batched_tokens, time.perf_counter() - t0, self.block_manager.utilization)
        return outputs

    def _take_pending(self):
        pending, self._pending = self._pending, None
        return pending

    @staticmethod
    def _needs_host_tokens(s: ScheduledRequest) -> bool:
        r = s.request
        start = r.num_computed_tokens
        if s.num_new_tokens == 1 and start == r.num_tokens - 1:
            return False  # a single newest token can come from the device
        return r.in_flight_within(start)

    def _launch(self, group: list[ScheduledRequest], previous) -> "_Pending | None":
        """engine.py:196-228: a portion that reaches the end of the known tokens asks for the
        logits of its last place and gets a token sampled; others ask for none."""
        items: list[BatchItem] = []
        sampled: list[Request] = []
        for s in group:
            r = s.request
            start = r.num_computed_tokens
            completes = start + s.num_new_tokens == r.num_tokens
            want = "last" if completes else "none"
            row = None
            if previous is not None and s.num_new_tokens == 1 and r.has_token_in_flight:
                row = previous.rows.get(r.request_id)
            if row is not None:
                items.append(BatchItem(r.request_id, [0], start, want, feedback_row=row))
            else:
                items.append(BatchItem(r.request_id, r.tokens(start, s.num_new_tokens), start, want))
            if completes:
                sampled.append(r)
        logits = self.runner.step(items)
        for s in group:
            s.request.num_computed_tokens += s.num_new_tokens
        if not sampled:
            return None
        keys = [r.stream_base + r.num_output_tokens for r in sampled]
        tokens = self.sampler.sample(logits, [r.sampling_params for r in sampled], keys)
        # tokens and the device's error flag (one buffer) go to pinned host memory behind the kernels, in one copy
        host = self._host_tokens[self._flip]
        self._flip ^= 1
        host.copy_(self.core.rt.status, non_blocking=True)
        event = self._events[self._flip]
        event.record()
        max_len = self.config.scheduler.max_model_len
        pending = _Pending(sampled, [r.launch_token() for r in sampled], host, event, {r.request_id: i for i, r in enumerate(sampled)})
        for r in sampled:
            # stops by count need no token value: decide them now, so the request is not run again
            if r.at_count_limit(max_len):
                self.scheduler.finish_request(r, FinishReason.LENGTH)
        return pending

    def _resolve(self, pending) -> list[RequestOutput]:
        """Read a launched step's tokens, put them in place of the placeholders, check stop
        tokens, report (engine.py:243-272)."""
        if pending is None:
            return []
        pending.event.synchronize()
        values = pending.host.tolist()  # the step's one device-to-host read: tokens in row order, then the error flag
        if values[-1]:
            self.core.rt.check_error_flag()
        outputs: list[RequestOutput] = []
        now = time.perf_counter()
        for r, idx, tok in zip(pending.sampled, pending.indices, values):
            if r.request_id in pending.skip or idx >= len(r.output_token_ids):
                continue  # stopped or aborted meanwhile: this token is not part of its output
            r.land_token(idx, tok, now)
            if r.stops_at(tok) and not (r.is_finished and r.finish_reason == FinishReason.STOP):
                # whatever was launched after it (the token of the step in flight) is dropped
                r.truncate_output(idx + 1)
                if not r.is_finished:
                    self.scheduler.finish_request(r, FinishReason.STOP)
                else:  # already closed by count in the same step: the stop token wins
                    r.finish_reason = FinishReason.STOP
                if self._pending is not None:
                    self._pending.skip.add(r.request_id)
            last = idx == len(r.output_token_ids) - 1
            finished = r.is_finished and last
            if finished:
                r.finish_time = now  # the request ends for its caller when its last token is on the host
                self.metrics.record_finished(r)
            elif not r.is_finished:
                self.block_manager.mark_computed(r.request_id, r.num_computed_tokens)
            out = RequestOutput(
                request_id=r.request_id,
                prompt_token_ids=r.prompt_token_ids,
                output_token_ids=[t for t in r.output_token_ids[: idx + 1]],
                new_token_ids=[tok],
                finished=finished,
                finish_reason=r.finish_reason if finished else None,
            )
            if self.tokenizer is not None:
                out.text = self.tokenizer.decode(out.output_token_ids)
            outputs.append(out)
        return outputs

    # ------------------------------------------------------------------ stats
    def stats(self) -> dict[str, Any]:
        """Figures of the run so far under the headings kvforge reports (engine.py:275-297):
        serving metrics, the cache's pages and bytes, the scheduler's queues, forward passes."""
        pages = self.block_manager.stats()
        per_page = self.kv_cache.bytes_per_block
        cache = asdict(pages)
        cache.update(bytes_total=self.kv_cache.memory_bytes, bytes_per_block=per_page, bytes_in_use=pages.num_used_blocks * per_page)
        queues = {key: getattr(self.scheduler, key) for key in ("num_running", "num_waiting", "num_preemptions")}
        return {
            "metrics": self.metrics.summary(),
            "kv_cache": cache,
            "scheduler": queues,
            "forward_passes": self.runner.num_forward_passes,
            "graphs_captured": len(self.runner.graph_kernels),
        }
