"""``InferenceEngine``: the Python entry point.  One ``step()`` is one scheduler decision,
one flat forward over everything scheduled, one sampling call, and the bookkeeping.

Names and meanings follow umarhassan-cloud/kvforge's ``InferenceEngine``
(src/tokenvault/engine.py:39-297): ``add_request``, ``abort_request``,
``has_unfinished_requests``, ``generate`` (outputs in prompt order), ``step``, ``stats``.
The model is given as a folder (``config.json`` + safetensors), or is made with random
weights from ``config.model`` and ``config.seed`` as kvforge does when it is given none
(engine.py:52-54).
"""

from __future__ import annotations

import itertools
import time
from collections.abc import Sequence
from dataclasses import asdict
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
from .tokenizer import Tokenizer


class InferenceEngine:
    def __init__(
        self,
        config: EngineConfig | None = None,
        model: str | Path | None = None,
        tokenizer: Tokenizer | None = None,
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
            cuda_graphs=config.cuda_graphs and config.dtype == torch.bfloat16,
        )
        self.block_manager = self.core.block_manager
        self.kv_cache = self.core.pool
        self.runner = self.core.runner
        self.sampler = Sampler(self.core.device, sc.max_num_seqs)
        self.scheduler = Scheduler(sc, self.block_manager, self.core.state_slots)
        self.metrics = MetricsCollector()
        self._ids = itertools.count()
        self.vocab_size = spec.vocab_size

    # ------------------------------------------------------------------ API
    def add_request(
        self,
        prompt: str | Sequence[int],
        sampling_params: SamplingParams | None = None,
        request_id: str | None = None,
        arrival_time: float | None = None,
    ) -> str:
        """engine.py:106-134."""
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("string prompts need a tokenizer")
            token_ids = self.tokenizer.encode(prompt)
        else:
            token_ids = [int(t) for t in prompt]
        if any(t < 0 or t >= self.vocab_size for t in token_ids):
            raise ValueError("prompt contains out-of-vocabulary token ids")
        request_id = request_id or f"req-{next(self._ids)}"
        eos = self.tokenizer.eos_token_id if self.tokenizer else self.core.spec.eos_token_id
        params = sampling_params or SamplingParams()
        req = Request(
            request_id=request_id,
            prompt_token_ids=token_ids,
            sampling_params=params,
            eos_token_id=eos,
            stream_base=request_stream_base(self.config.seed, request_id, params),
        )
        if arrival_time is not None:
            req.arrival_time = arrival_time
        self.scheduler.add_request(req)
        return request_id

    def abort_request(self, request_id: str) -> bool:
        req = self.scheduler.abort_request(request_id)
        if req is not None:
            self.metrics.record_finished(req)
        return req is not None

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    def generate(
        self,
        prompts: Sequence[str | Sequence[int]],
        sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
    ) -> list[RequestOutput]:
        """Offline batch generation; outputs in prompt order (engine.py:145-159)."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        done: dict[str, RequestOutput] = {}
        while self.has_unfinished_requests():
            for out in self.step():
                if out.finished:
                    done[out.request_id] = out
        return [done[i] for i in ids if i in done]

    # ------------------------------------------------------------------ step
    def step(self) -> list[RequestOutput]:
        t0 = time.perf_counter()
        sched = self.scheduler.schedule()
        if sched.is_empty:
            return []
        new_tokens = self._run(sched.scheduled)
        outputs = self._postprocess(sched.scheduled, new_tokens)
        self.metrics.record_step(len(sched.scheduled), sched.num_batched_tokens, time.perf_counter() - t0, self.block_manager.utilization)
        return outputs

    def _run(self, group: list[ScheduledRequest]) -> dict[str, int]:
        """engine.py:196-228: a portion that reaches the end of the known tokens asks for the
        logits of its last place and gets a token sampled; others ask for none."""
        items: list[BatchItem] = []
        sampled: list[Request] = []
        for s in group:
            r = s.request
            start = r.num_computed_tokens
            completes = start + s.num_new_tokens == r.num_tokens
            items.append(BatchItem(r.request_id, r.all_token_ids[start : start + s.num_new_tokens], start, "last" if completes else "none"))
            if completes:
                sampled.append(r)
        logits = self.runner.step(items)
        for s in group:
            s.request.num_computed_tokens += s.num_new_tokens
        out: dict[str, int] = {}
        if sampled:
            keys = [r.stream_base + r.num_output_tokens for r in sampled]
            tokens = self.sampler.sample(logits, [r.sampling_params for r in sampled], keys)
            host = tokens.tolist()  # the step's one device-to-host read
            self.core.rt.check_error_flag()
            for r, t in zip(sampled, host):
                out[r.request_id] = t
        return out

    def _postprocess(self, scheduled: list[ScheduledRequest], new_tokens: dict[str, int]) -> list[RequestOutput]:
        """engine.py:243-272."""
        now = time.perf_counter()
        max_len = self.config.scheduler.max_model_len
        outputs: list[RequestOutput] = []
        for s in scheduled:
            r = s.request
            emitted: list[int] = []
            reason: FinishReason | None = None
            if r.request_id in new_tokens:
                t = new_tokens[r.request_id]
                r.append_token(t, now)
                emitted.append(t)
                reason = r.check_stop(max_len)
            if reason is not None:
                self.scheduler.finish_request(r, reason)
                self.metrics.record_finished(r)
            else:
                self.block_manager.mark_computed(r.request_id, r.num_computed_tokens)
            if emitted or r.is_finished:
                out = RequestOutput.from_request(r, emitted)
                if self.tokenizer is not None:
                    out.text = self.tokenizer.decode(out.output_token_ids)
                outputs.append(out)
        return outputs

    # ------------------------------------------------------------------ stats
    def stats(self) -> dict[str, Any]:
        """engine.py:275-297."""
        bm = self.block_manager.stats()
        return {
            "metrics": self.metrics.summary(),
            "kv_cache": {
                **asdict(bm),
                "bytes_total": self.kv_cache.memory_bytes,
                "bytes_per_block": self.kv_cache.bytes_per_block,
                "bytes_in_use": bm.num_used_blocks * self.kv_cache.bytes_per_block,
            },
            "scheduler": {
                "num_running": self.scheduler.num_running,
                "num_waiting": self.scheduler.num_waiting,
                "num_preemptions": self.scheduler.num_preemptions,
            },
            "forward_passes": self.runner.num_forward_passes,
        }
