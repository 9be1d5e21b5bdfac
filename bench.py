"""Decode and prefill throughput of the Llama-3.2-1B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of a batch of 8 requests.  The K timed steps are spread evenly over
contexts from 2,048 to 4,096 tokens (a request decoding from a 2,048-token prompt to 4,096 sees
each of them once), so ``value``, decoded tokens a second, is the mean over that range; it is
timed on the device with CUDA events around exactly K steps of the step function plus the
sampling kernel.  ``e2e`` is the same through ``InferenceEngine`` (scheduler, token ids from
and to the host every step) with prompts whose lengths are spread over the same range.  The
same line carries a 2,048-token prefill, the decode step's HBM roofline fraction, and under
``points`` decode at batch 1 and 64 (same spread), batch 8 at the two ends of the range, the
true 32-bit path, a mixed step of the 3B shape and a serving load of the 8B shape.
One JSON line on stdout.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 2048
CONTEXT = 4096
PREFILL_TOKENS = 2048


def peaks() -> dict:
    """Measured peaks from ``MEASURED_PEAKS.json`` beside this file if it is there, else
    fallback figures of an earlier measurement of a B200 (a copy's bandwidth, cuBLAS bfloat16)."""
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            for k in ("hbm_gbs", "bf16_tflops"):
                if isinstance(data.get(k), (int, float)) and data[k] > 0:
                    out[k] = float(data[k])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu: str = "0") -> None:
        self.proc = None
        self.gpu = gpu

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text, _ = self.proc.communicate()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in text.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max_clock,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def model_numbers(cfg, layers: int) -> dict:
    """Bytes and flops of the shape (bfloat16 weights)."""
    h, d, nh, nkv, inter, v = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size, cfg.vocab_size
    per_layer = h * d * (nh + 2 * nkv) + nh * d * h + 3 * h * inter
    head = v * h
    return {
        "weight_bytes": 2 * (layers * per_layer + head),  # every weight a decode step reads once
        "kv_bytes_per_token": 2 * layers * nkv * d * 2,
        "linear_flops_per_token": 2 * layers * per_layer,
        "head_flops_per_row": 2 * head,
        "attn_flops_causal": lambda t: layers * 4 * nh * d * t * (t + 1) // 2,
    }


def make_core(cfg, batch: int, max_tokens: int, ctx_cap: int, cuda_graphs: bool = True, dtype: str = "bfloat16"):
    from kvforge_b200.config.engine_config import CacheConfig
    from kvforge_b200.engine.core import EngineCore, spec_from_config

    blocks = batch * (-(-ctx_cap // 16)) + 8
    return EngineCore(
        spec_from_config(cfg), dtype=dtype, seed=0,
        cache=CacheConfig(block_size=16, num_blocks=blocks, watermark=0.0),
        max_num_seqs=batch, max_num_batched_tokens=max_tokens, max_model_len=ctx_cap, cuda_graphs=cuda_graphs,
    )  # fmt: skip


def spread(n: int, lo: int, hi: int) -> list[int]:
    """``n`` contexts from ``lo`` to ``hi`` (the tokens a cache holds before the step), evenly spaced."""
    if n == 1:
        return [(lo + hi) // 2]
    return [lo + round(i * (hi - lo) / (n - 1)) for i in range(n)]


def time_decode(core, batch: int, contexts: list[int], warmup: int, sample: bool = True):
    """Decode steps of ``batch`` requests on synthetic keys and values: step ``i`` finds
    ``contexts[i]`` tokens in every cache and adds one.  The first ``warmup`` steps are untimed.
    Returns (seconds of the timed steps, kernels launched in them, their mean context)."""
    import torch

    from kvforge_b200.engine.step import BatchItem
    from kvforge_b200.sampling.params import SamplingParams
    from kvforge_b200.sampling.sampler import Sampler

    bm = core.block_manager
    ids = [f"b{i}" for i in range(batch)]
    for rid in ids:
        bm.allocate(rid, max(contexts) + 1)
        core.state_slots.allocate(rid)
    for t in core.pool.k + core.pool.v:  # synthetic cache contents
        t.normal_(0.0, 0.5)
    sampler = Sampler(core.device, batch)
    params = [SamplingParams(temperature=0.0)] * batch
    gen = torch.Generator().manual_seed(0)
    vocab = core.spec.vocab_size
    tokens = torch.randint(0, vocab, (len(contexts), batch), generator=gen).tolist()

    def one(i):
        logits = core.runner.step([BatchItem(rid, [tokens[i][j]], contexts[i], "last") for j, rid in enumerate(ids)])
        if sample:
            sampler.sample(logits, params, [0] * batch)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    from kvforge_b200 import ops

    k0 = ops.launch_count + core.runner.num_graph_kernels
    g0 = sum(core.runner.graph_kernels.values())
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, len(contexts)):
        one(i)
    end.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(end) / 1e3
    # kernels of this library: launched one by one (sampling; the model's when graphs are off) plus
    # those inside replayed graphs
    launched = ops.launch_count + core.runner.num_graph_kernels - k0
    if sum(core.runner.graph_kernels.values()) != g0:
        launched = None  # a graph was captured inside the timed region: the count would mix things
    for rid in ids:
        bm.free(rid)
        core.state_slots.free(rid)
    timed = contexts[warmup:]
    return seconds, launched, sum(timed) / len(timed) + 1


def decode_schedule(steps: int, warmup: int, lo: int = PROMPT_LEN, hi: int = CONTEXT - 1) -> list[int]:
    """Warm-up steps at both ends of the range (so that every graph the timed steps replay exists),
    then ``steps`` contexts spread over it."""
    ends = [lo, hi, (lo + hi) // 2]
    return [ends[i % 3] for i in range(warmup)] + spread(steps, lo, hi)


def time_prefill(core, tokens: int, reps: int = 3):
    import torch

    from kvforge_b200.engine.step import BatchItem

    gen = torch.Generator().manual_seed(1)
    # host token ids as an int32 array, which is how the engine hands a portion of a prompt to the step function
    prompt = torch.randint(0, core.spec.vocab_size, (tokens,), generator=gen).to(torch.int32).numpy()
    times = []
    for _ in range(reps + 1):
        core.block_manager.allocate("p", tokens)
        core.state_slots.allocate("p")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        core.runner.step([BatchItem("p", prompt, 0, "last")])
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / 1e3)
        core.block_manager.free("p")
        core.state_slots.free("p")
    return min(times[1:])


def time_mixed(core, decodes: int, context: int, chunk: int, reps: int = 5):
    """A mixed step: ``decodes`` requests with ``context`` tokens in their caches bring one token
    each, beside one request that brings a portion of ``chunk`` prompt tokens (from position 0).
    Returns the seconds per step of ``reps`` steps run back to back (the host prepares a step
    while the device runs the one before)."""
    import torch

    from kvforge_b200.engine.step import BatchItem

    bm = core.block_manager
    ids = [f"d{i}" for i in range(decodes)]
    for rid in ids:
        bm.allocate(rid, context)
        core.state_slots.allocate(rid)
    for t in core.pool.k + core.pool.v:  # synthetic cache contents
        t.normal_(0.0, 0.5)
    gen = torch.Generator().manual_seed(3)
    vocab = core.spec.vocab_size
    prompt = torch.randint(0, vocab, (chunk,), generator=gen).tolist()
    pos = context
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(reps + 2):  # two untimed steps (the second replays what the first captured), then the timed ones back to back
        if i == 2:
            torch.cuda.synchronize()
            start.record()
        for rid in ids:
            bm.append_slots(rid, pos + 1, pos)
        bm.allocate("p", chunk)
        core.state_slots.allocate("p")
        items = [BatchItem(rid, [int(torch.randint(0, vocab, (1,), generator=gen))], pos, "last") for rid in ids]
        items.append(BatchItem("p", prompt, 0, "last"))
        core.runner.step(items)
        bm.free("p")
        core.state_slots.free("p")
        pos += 1
    end.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(end) / 1e3 / reps
    for rid in ids:
        bm.free(rid)
        core.state_slots.free(rid)
    return seconds


def time_e2e(cfg, batch: int, steps: int, warmup: int):
    """The same decode steps through ``InferenceEngine``: prompts of 2,048 host token ids in,
    a token id per request out to the host every step."""
    import torch

    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    blocks = batch * (CONTEXT // 16) + 8
    engine = InferenceEngine(
        EngineConfig(
            model=cfg, cache=CacheConfig(block_size=16, num_blocks=blocks, watermark=0.0),
            scheduler=SchedulerConfig(max_num_seqs=batch, max_num_batched_tokens=PREFILL_TOKENS, max_model_len=CONTEXT),
            dtype="bfloat16", seed=0,
        )
    )  # fmt: skip
    gen = torch.Generator().manual_seed(2)
    # A short timed region (a few dozen steps are some 20 ms) is at the mercy of one hiccup of the host: it
    # is then taken three times, each time exactly ``steps`` steps, and the median counts.
    reps = 3 if steps <= 48 else 1
    # requests whose prompts are done decode while the others are still in theirs: leave room
    room = warmup + reps * (steps + 3) + 2 * batch + 12
    sp = SamplingParams(max_tokens=room, temperature=0.0, ignore_eos=True)
    # prompt lengths spread over the range, so the batch's mean context is that of the device-timed steps
    for n in spread(batch, PROMPT_LEN, CONTEXT - room - 1):
        engine.add_request(torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist(), sp)
    while any(r.is_prefill for r in engine.scheduler.requests.values()):
        engine.step()
    for _ in range(warmup):
        engine.step()
    rates, h2d, timed = [], 0, 0
    for _ in range(reps):
        torch.cuda.synchronize()
        # The engine reads a step's tokens while the next step runs, so a call of step() hands out the tokens of
        # the step before.  A few untimed calls after the synchronize put a step in flight and let host and device
        # fall into step; each of the K timed calls then copies its step's inputs to the device, launches it, and
        # reads the tokens of the step before it from the device: K steps' worth of work and of results, without the
        # one-off filling and draining of that pipeline.
        for _ in range(3):
            engine.step()
        h0 = engine.runner.h2d_bytes
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        produced = 0
        for _ in range(steps):
            produced += sum(len(o.new_token_ids) for o in engine.step())
        end.record()
        wall = time.perf_counter() - t0  # the K-th call has returned: K x batch tokens are on the host
        torch.cuda.synchronize()
        seconds = max(start.elapsed_time(end) / 1e3, wall)
        assert produced == batch * steps, (produced, batch * steps)
        rates.append(produced / seconds)
        h2d += engine.runner.h2d_bytes - h0
        timed += steps
    rates.sort()
    return rates[len(rates) // 2], h2d / timed, 4 * batch + 4  # token ids and the error flag


def run_own(args) -> dict:
    import torch

    from kvforge_b200 import PRESETS

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    cfg = PRESETS["llama-3.2-1b"]
    layers = cfg.num_layers
    pk = peaks()
    nums = model_numbers(cfg, layers)
    batch = 8
    ctx_cap = CONTEXT

    core = make_core(cfg, 64, PREFILL_TOKENS, ctx_cap)
    try:
        gpu = "GPU-" + str(torch.cuda.get_device_properties(0).uuid)
    except Exception:  # an older torch without the uuid field
        gpu = "0"
    sampler = ClockSampler(gpu)
    sampler.start()
    seconds, launches, mean_ctx = time_decode(core, batch, decode_schedule(args.steps, args.warmup), args.warmup)
    clocks = sampler.stop()
    tok_s = batch * args.steps / seconds
    step_bytes = nums["weight_bytes"] + batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (seconds / args.steps) / 1e9

    points = {}
    k = max(16, args.steps // 2)
    w = max(3, args.warmup)
    for b in (1, 64):
        sec, _, _ = time_decode(core, b, decode_schedule(k, w), w)
        points[f"decode_b{b}"] = round(b * k / sec, 1)
    # the two ends of the range at batch 8: contexts of 2,048 and of 4,095 tokens, advancing by one a step
    for name, lo in (("decode_b8_ctx2048", PROMPT_LEN), ("decode_b8_ctx4096", CONTEXT - 1 - k - w)):
        sec, _, _ = time_decode(core, batch, [lo + i for i in range(w + k)], w)
        points[name] = round(batch * k / sec, 1)

    p_seconds = time_prefill(core, PREFILL_TOKENS)
    p_flops = PREFILL_TOKENS * nums["linear_flops_per_token"] + nums["head_flops_per_row"] + nums["attn_flops_causal"](PREFILL_TOKENS)
    del core
    torch.cuda.empty_cache()

    e2e_tok_s, h2d, d2h = time_e2e(cfg, batch, args.steps, args.warmup)
    torch.cuda.empty_cache()

    # the true 32-bit path of the same shape (FFMA products, no tensor cores): a figure for the record
    core = make_core(cfg, batch, PREFILL_TOKENS, ctx_cap, dtype="float32")
    k32 = 8
    sec, _, _ = time_decode(core, batch, decode_schedule(k32, 3), 3)
    points["decode_b8_float32"] = round(batch * k32 / sec, 1)
    points["prefill_float32"] = round(PREFILL_TOKENS / time_prefill(core, PREFILL_TOKENS, reps=1), 1)
    del core
    torch.cuda.empty_cache()

    # Llama-3.2-3B shape: one mixed step, 32 requests decoding at context 2,048 beside a 1,024-token portion of a prompt
    cfg3 = PRESETS["llama-3.2-3b"]
    core = make_core(cfg3, 33, PREFILL_TOKENS, ctx_cap)
    points["mixed_step_3b_ms"] = round(1e3 * time_mixed(core, 32, 2048, 1024), 3)
    del core
    torch.cuda.empty_cache()

    # Llama-3.1-8B shape: 64 requests, prompts of 128 to 2,048 tokens, 256 generated each, through the entry point
    load = run_load(PRESETS["llama-3.1-8b"], 64)
    points["load_8b_generated_tok_s"] = load["generated_tokens_per_s"]
    points["load_8b_total_tok_s"] = load["total_tokens_per_s"]
    torch.cuda.empty_cache()

    return {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B shape, mean over contexts 2048->4096)",
        "value": round(tok_s, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(1e3 * seconds / args.steps, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (random token ids, random-init weights, synthetic cache contents for the device-timed decode)",
        "impl": "kvforge_b200",
        "config": {
            "model": "llama-3.2-1b-shape",
            "layers": layers,
            "layers_of_model": cfg.num_layers,
            "hidden": cfg.hidden_size,
            "heads": cfg.num_heads,
            "kv_heads": cfg.num_kv_heads,
            "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size,
            "global_batch": batch,
            "seq_len": CONTEXT,
            "prompt_len": PROMPT_LEN,
            "mean_context": round(mean_ctx, 1),
            "kv_block_size": 16,
            "tied_embeddings": cfg.tie_word_embeddings,
            "rope": "theta 5e5, llama3 x32",
            "l2": "inputs larger than L2: every step streams 2.47 GB of weights",
            "peaks": pk["source"],
            "points_3b": "llama-3.2-3b shape, 28 layers: 32 decoding at context 2048 + one 1024-token prompt portion, one step",
            "points_8b": "llama-3.1-8b shape, 32 layers: 64 requests, prompts U[128,2048], 256 tokens each, 2048-token budget",
        },
        "e2e": {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": launches,
        "prefill": {
            "value": round(PREFILL_TOKENS / p_seconds, 1),
            "tokens": PREFILL_TOKENS,
            "ms": round(1e3 * p_seconds, 3),
            "frac": round(p_flops / p_seconds / (pk["bf16_tflops"] * 1e12), 4),
        },
        "roofline": {
            "bound": "hbm",
            "achieved": round(achieved, 1),
            "peak": pk["hbm_gbs"],
            "unit": "GB/s",
            "frac": round(achieved / pk["hbm_gbs"], 4),
        },
        "points": points,
        "clocks": clocks,
    }


def _graph_time(fn, calls: int, reps: int) -> float:
    """Seconds per call of ``fn(i)``, ``calls`` of them captured in one CUDA graph (so that
    launch overhead of the host does not count) and replayed ``reps`` times."""
    import torch

    for i in range(2):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(calls):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / 1e3 / (reps * calls)


def run_kernel_only(args, cfg) -> dict:
    """A single kernel of the decode step on the 1B shape, on inputs larger than L2 (several
    copies of the weights or of the cache are cycled through)."""
    import torch

    from kvforge_b200 import ops

    pk = peaks()
    dev = "cuda"
    nh, nkv, d, bs = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, args.block_size
    if args.only == "attention":
        b, ctx = args.batch, args.context
        nblk = b * (-(-ctx // bs))
        copies = max(2, min(8, int(1.5e9 // max(1, nblk * nkv * bs * d * 4))))
        kcs = [torch.randn(nblk, nkv, bs, d, device=dev).bfloat16() for _ in range(copies)]
        vcs = [torch.randn(nblk, nkv, bs, d, device=dev).bfloat16() for _ in range(copies)]
        tables = torch.randperm(nblk, device=dev).int().view(b, -1).contiguous()
        q = torch.randn(b, nh * d, device=dev).bfloat16()
        out = torch.empty(b, nh * d, device=dev, dtype=torch.bfloat16)
        qsl = torch.arange(b + 1, device=dev, dtype=torch.int32)
        cl = torch.full((b,), ctx, device=dev, dtype=torch.int32)
        from kvforge_b200.parts.attention import CLUSTER_MERGE_MAX_PAIRS

        # --split 0: the engine's choice, the launch's size and the kernel's own lengthening of it
        split = args.split or ops.attention_split_size(b, nkv, ctx, reach=ctx, head_dim=d)
        wave = 0 if args.split else ops.attention_wave_target(b, nkv, d)
        sa, sm = ops.attention_scratch_shapes(b, nh, d, ctx, split)
        scratch = (torch.empty(sa, device=dev), torch.empty(sm, device=dev), torch.zeros(b * nkv, dtype=torch.int32, device=dev))
        sec = _graph_time(
            lambda i: ops.paged_attention(q, out, kcs[i % copies], vcs[i % copies], tables, qsl, cl, b, 1, nh, nkv, d,
                                          d**-0.5, scratch=scratch, max_context=ctx, split_size=split, wave_target=wave,
                                          cluster=b * nkv <= CLUSTER_MERGE_MAX_PAIRS),  # as the attention part chooses
            calls=max(2, args.steps), reps=3,
        )  # fmt: skip
        nbytes = b * ctx * 2 * nkv * d * 2
        return {"only": "attention", "batch": b, "context": ctx, "split": split, "us": round(sec * 1e6, 2),
                "GB/s": round(nbytes / sec / 1e9, 1), "frac_of_hbm_peak": round(nbytes / sec / 1e9 / pk["hbm_gbs"], 3)}  # fmt: skip
    if args.only == "attention-prefill":
        # one prompt of `context` tokens, all of them queries (the kernel of prompts and mixed batches)
        ctx = args.context
        nblk = -(-ctx // bs)
        kc = torch.randn(nblk, nkv, bs, d, device=dev).bfloat16()
        vc = torch.randn(nblk, nkv, bs, d, device=dev).bfloat16()
        tables = torch.randperm(nblk, device=dev).int().view(1, -1).contiguous()
        q = torch.randn(ctx, nh * d, device=dev).bfloat16()
        out = torch.empty(ctx, nh * d, device=dev, dtype=torch.bfloat16)
        qsl = torch.tensor([0, ctx], device=dev, dtype=torch.int32)
        cl = torch.tensor([ctx], device=dev, dtype=torch.int32)
        err = torch.zeros(4, device=dev, dtype=torch.int32)
        sec = _graph_time(
            lambda i: ops.paged_attention(q, out, kc, vc, tables, qsl, cl, 1, ctx, nh, nkv, d, d**-0.5, err=err),
            calls=max(2, args.steps), reps=3,
        )  # fmt: skip
        if int(err.sum()):
            raise SystemExit("the attention kernel raised its error flag")
        flops = 4 * nh * d * ctx * (ctx + 1) // 2
        return {"only": "attention-prefill", "tokens": ctx, "us": round(sec * 1e6, 2), "TFLOP/s": round(flops / sec / 1e12, 1),
                "frac_of_bf16_peak": round(flops / sec / 1e12 / pk["bf16_tflops"], 3)}  # fmt: skip
    if args.only == "sample":
        # one token per row of float logits [batch, vocabulary]; copies are cycled so that rows come from HBM
        r, v = args.batch, cfg.vocab_size
        copies = max(2, min(16, int(4e8 // (r * v * 4)) + 1))
        if args.peaked:  # a few likely tokens and a long tail (logit = -1.5 ln(rank) + noise), as a trained model's rows are
            ranks = torch.stack([torch.randperm(v, device=dev) for _ in range(r)]).float()
            logits = [-1.5 * torch.log1p(ranks) + 0.3 * torch.randn(r, v, device=dev) for _ in range(copies)]
        else:
            logits = [torch.randn(r, v, device=dev) * 3 for _ in range(copies)]
        out = torch.empty(r, device=dev, dtype=torch.int32)
        temps = torch.full((r,), args.temperature, device=dev)
        ks = torch.full((r,), args.top_k, device=dev, dtype=torch.int32)
        ps = torch.full((r,), args.top_p, device=dev)
        keys = torch.arange(r, device=dev, dtype=torch.int64)
        sec = _graph_time(lambda i: ops.sample(logits[i % copies], out, temps, ks, ps, keys), calls=max(2, args.steps), reps=3)
        nbytes = r * v * 4
        return {"only": "sample", "rows": r, "vocab": v, "temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p,
                "us": round(sec * 1e6, 2), "GB/s_one_pass": round(nbytes / sec / 1e9, 1)}  # fmt: skip
    shapes = {"qkv": ((nh + 2 * nkv) * d, cfg.hidden_size), "o": (cfg.hidden_size, nh * d),
              "gate_up": (2 * cfg.intermediate_size, cfg.hidden_size), "down": (cfg.hidden_size, cfg.intermediate_size),
              "lm_head": (cfg.vocab_size, cfg.hidden_size)}  # fmt: skip
    n, k = shapes[args.shape]
    m = args.batch
    copies = max(2, min(12, int(1.2e9 // (n * k * 2))))
    ws = [(torch.randn(n, k, device=dev) * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(m, k, device=dev).bfloat16()
    splits = ops.skinny_splits(n, k, m)
    out = ops.Partials(torch.empty(splits, m, n, device=dev)) if splits > 1 else torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    sec = _graph_time(lambda i: ops.gemm_skinny(x, ws[i % copies], out), calls=max(2, args.steps), reps=3)
    nbytes = n * k * 2
    return {"only": "gemm", "shape": args.shape, "M": m, "N": n, "K": k, "splits": splits, "us": round(sec * 1e6, 2),
            "GB/s": round(nbytes / sec / 1e9, 1), "frac_of_hbm_peak": round(nbytes / sec / 1e9 / pk["hbm_gbs"], 3)}  # fmt: skip


def run_load(cfg, nreq: int, short_prompts: bool = False) -> dict:
    """A serving load through the Python entry point: ``nreq`` requests with prompt lengths drawn
    uniformly from 128 to 2,048 and 256 greedy tokens each, under chunked prefill with a
    2,048-token budget."""
    import random
    import time

    import torch

    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    rng = random.Random(0)
    if short_prompts:
        # many short requests that end at different times: most steps are a batch of decoding
        # requests beside the short prompt of one that was just admitted
        prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(16, 256))] for _ in range(nreq)]
        params = [SamplingParams(max_tokens=rng.randint(16, 128), temperature=0.0, ignore_eos=True) for _ in prompts]
    else:
        prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(128, 2048))] for _ in range(nreq)]
        params = [SamplingParams(max_tokens=256, temperature=0.0, ignore_eos=True)] * nreq
    engine = InferenceEngine(EngineConfig(
        model=cfg, cache=CacheConfig(block_size=16, num_blocks=None, kv_cache_memory_gb=16.0),
        scheduler=SchedulerConfig(max_num_seqs=64, max_num_batched_tokens=PREFILL_TOKENS, max_model_len=CONTEXT), dtype="bfloat16",
    ))  # fmt: skip
    # the same load twice untimed: every graph the timed pass replays exists by then (a shape of
    # many tokens is captured at its second coming)
    for _ in range(2):
        engine.generate(prompts, params)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_in, n_out = sum(len(q) for q in prompts), sum(len(o.output_token_ids) for o in outs)
    stats = engine.stats()
    m = stats["metrics"]
    del engine
    return {"only": "load", "requests": nreq, "prompt_tokens": n_in, "generated_tokens": n_out,
            "seconds": round(dt, 3), "generated_tokens_per_s": round(n_out / dt, 1), "total_tokens_per_s": round((n_in + n_out) / dt, 1),
            "tpot_p50_ms": round(m["tpot_p50_ms"], 3), "preemptions": stats["scheduler"]["num_preemptions"]}  # fmt: skip


def run_only(args) -> dict:
    """One part alone on a small footing: what the profiler is pointed at."""
    from kvforge_b200 import PRESETS

    cfg = PRESETS[args.preset]
    if args.only == "load":
        nreq = args.batch if args.batch != 8 else (256 if args.short_prompts else 64)
        return {"preset": args.preset, **run_load(cfg, nreq, args.short_prompts)}
    if args.only in ("attention", "attention-prefill", "gemm", "sample"):
        return run_kernel_only(args, cfg)
    ctx_cap = max(CONTEXT, args.context + args.steps + args.warmup + 16)
    core = make_core(cfg, max(args.batch, 1) + (args.only == "mixed"), PREFILL_TOKENS, ctx_cap, cuda_graphs=not args.no_graphs)
    if args.only == "decode":
        seconds, launches, mean_ctx = time_decode(core, args.batch, [args.context + i for i in range(args.warmup + args.steps)], args.warmup)
        return {"only": "decode", "batch": args.batch, "context": mean_ctx, "ms_per_step": round(1e3 * seconds / args.steps, 4),
                "tokens_per_s": round(args.batch * args.steps / seconds, 1), "gpu_launches": launches}  # fmt: skip
    if args.only == "mixed":
        chunk = 1024
        seconds = time_mixed(core, args.batch, args.context, chunk)
        return {"only": "mixed", "preset": args.preset, "decode_requests": args.batch, "context": args.context, "prompt_portion": chunk,
                "ms": round(1e3 * seconds, 3), "tokens_per_s": round((args.batch + chunk) / seconds, 1)}  # fmt: skip
    seconds = time_prefill(core, PREFILL_TOKENS, reps=max(1, args.steps))
    return {"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(1e3 * seconds, 3), "tokens_per_s": round(PREFILL_TOKENS / seconds, 1)}


REF_DIR = ROOT / "baseline" / "_ref"


def _reference_package() -> str | None:
    """Puts umarhassan-cloud/kvforge's package (``tokenvault``) on the path.  It is pure Python:
    what a wheel of it would install is a copy of its ``src/tokenvault`` folder, and that copy is
    what ``baseline/_ref/tokenvault`` holds (its build backend, hatchling, is not installed
    offline, so pip cannot make the wheel).  Returns why it is not there, or ``None``."""
    if not (REF_DIR / "tokenvault" / "__init__.py").is_file():
        # the checkout beside this repository (``../reference``), or wherever KVFORGE_REFERENCE_SRC points
        src = Path(os.environ.get("KVFORGE_REFERENCE_SRC", str(ROOT.parent / "reference" / "src"))) / "tokenvault"
        if not src.is_dir():
            return f"no copy of the reference package under {REF_DIR.relative_to(ROOT)} and no checkout at {src.parent} to copy it from"
        import shutil

        REF_DIR.mkdir(parents=True, exist_ok=True)
        shutil.copytree(src, REF_DIR / "tokenvault", ignore=shutil.ignore_patterns("__pycache__"))
    sys.path.insert(0, str(REF_DIR))
    return None


def run_reference(args) -> dict:
    """The same measurement on umarhassan-cloud/kvforge itself, unmodified, through its public
    API: ``tokenvault.InferenceEngine`` on ``cuda`` in bfloat16 at its own ``llama-1b`` preset
    (the Llama-3.2-1B shape; it has no llama3 frequency scaling, which changes neither bytes nor
    flops), pages of 16 tokens, 8 prompts of 2,048 random token ids, the same warm-up and step
    count.  ``e2e`` is ``InferenceEngine.step`` (host token ids in, host token ids out);
    ``value`` is its step function and sampler alone (``ModelRunner.execute`` + ``Sampler``),
    the counterpart of the own arm's device-timed figure.  Nothing of kvforge_b200 is imported."""
    why = _reference_package()
    if why:
        return {"impl": "reference", "unavailable": why}
    try:
        import torch
        import tokenvault
        from tokenvault import CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig
        from tokenvault.batching.continuous import BatchItem
        from tokenvault.model_loader import PRESETS as REF_PRESETS
    except Exception as e:  # the copy is there but does not import here
        return {"impl": "reference", "unavailable": f"importing the reference failed: {type(e).__name__}: {e}"}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    try:
        return _time_reference(args, torch, InferenceEngine, EngineConfig, CacheConfig, SchedulerConfig, SamplingParams, BatchItem, REF_PRESETS["llama-1b"], tokenvault.__file__)
    except Exception as e:
        return {"impl": "reference", "unavailable": f"the reference failed on this device: {type(e).__name__}: {str(e)[:300]}"}


def _time_reference(args, torch, InferenceEngine, EngineConfig, CacheConfig, SchedulerConfig, SamplingParams, BatchItem, cfg, where) -> dict:
    batch, steps, warmup = 8, args.steps, args.warmup
    pk = peaks()

    def engine_for(n_seqs: int):
        blocks = n_seqs * (CONTEXT // 16) + 8
        return InferenceEngine(EngineConfig(
            model=cfg, cache=CacheConfig(block_size=16, num_blocks=blocks, watermark=0.0),
            scheduler=SchedulerConfig(max_num_seqs=n_seqs, max_num_batched_tokens=PREFILL_TOKENS, max_model_len=CONTEXT),
            device="cuda", dtype=torch.bfloat16, seed=0,
        ))  # fmt: skip

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    gen = torch.Generator().manual_seed(2)
    engine = engine_for(batch)
    room = warmup + steps + 2 * batch + 12
    sp = SamplingParams(max_tokens=room, temperature=0.0, ignore_eos=True)
    # prompt lengths spread over 2,048 -> 4,096 like the own arm's, so both see the same mean context
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in spread(batch, PROMPT_LEN, CONTEXT - room - 1)]

    # prefill of one 2,048-token prompt through the step function, as the own arm times it
    bm = engine.block_manager
    p_times = []
    for _ in range(3):
        bm.allocate("p", prompts[0][:PREFILL_TOKENS])
        torch.cuda.synchronize()
        a, b = events()
        a.record()
        engine.runner.execute([BatchItem("p", prompts[0][:PREFILL_TOKENS], 0, "last")])
        b.record()
        torch.cuda.synchronize()
        p_times.append(a.elapsed_time(b) / 1e3)
        bm.free("p")
    p_seconds = min(p_times[1:])

    # end to end: the engine's own loop
    for prompt in prompts:
        engine.add_request(prompt, sp)
    while any(r.is_prefill for r in engine.scheduler.running) or engine.scheduler.num_waiting:
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    for _ in range(3):  # as in the own arm (the reference reads its tokens in the same call, so this changes nothing for it)
        engine.step()
    sampler = ClockSampler()
    sampler.start()
    a, b = events()
    t0 = time.perf_counter()
    a.record()
    produced = 0
    for _ in range(steps):
        produced += sum(len(o.new_token_ids) for o in engine.step())
    b.record()
    wall = time.perf_counter() - t0
    torch.cuda.synchronize()
    clocks = sampler.stop()
    e2e_seconds = max(a.elapsed_time(b) / 1e3, wall)
    assert produced == batch * steps, (produced, batch * steps)
    ctx_now = engine.scheduler.running[0].num_tokens
    width = -(-ctx_now // 16)
    # what its prepare_inputs copies per step (int64 tensors made from host lists) and what comes back
    h2d = 8 * (6 * batch + 1 + batch * width)
    d2h = 8 * batch
    for r in list(engine.scheduler.running):
        engine.abort_request(r.request_id)

    # the step function and the sampler alone, at batch 8 / 1 / 64
    def decode(n_seqs: int, k: int, w: int) -> tuple[float, float]:
        """Seconds per step and mean context of ``k`` timed steps spread over contexts 2,048 -> 4,096."""
        eng = engine if n_seqs <= batch else engine_for(n_seqs)
        ids = [f"d{i}" for i in range(n_seqs)]
        contexts = decode_schedule(k, w)
        filler = [1] * (max(contexts) + 1)
        for rid in ids:
            eng.block_manager.allocate(rid, filler)
        for c in eng.kv_cache.key_caches + eng.kv_cache.value_caches:
            c.normal_(0.0, 0.5)  # synthetic cache contents
        params = [SamplingParams(temperature=0.0)] * n_seqs
        a, b = events()
        for i, pos in enumerate(contexts):
            if i == w:
                torch.cuda.synchronize()
                a.record()
            logits = eng.runner.execute([BatchItem(rid, [7 + i], pos, "last") for rid in ids])
            eng.sampler(logits, params)
        b.record()
        torch.cuda.synchronize()
        for rid in ids:
            eng.block_manager.free(rid)
        return a.elapsed_time(b) / 1e3 / k, sum(contexts[w:]) / k + 1

    step_s, mean_ctx = decode(batch, steps, warmup)
    k = max(16, steps // 2)
    points = {"decode_b1": round(1 / decode(1, k, 3)[0], 1), "decode_b64": round(64 / decode(64, k, 3)[0], 1)}
    layers = cfg.num_layers
    h, d, nh, nkv, inter, v = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size, cfg.vocab_size
    per_layer = h * d * (nh + 2 * nkv) + nh * d * h + 3 * h * inter
    weight_bytes = 2 * (layers * per_layer + v * h)
    achieved = (weight_bytes + batch * mean_ctx * 2 * layers * nkv * d * 2) / step_s / 1e9
    p_flops = PREFILL_TOKENS * 2 * layers * per_layer + 2 * v * h + layers * 4 * nh * d * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2
    return {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B shape, mean over contexts 2048->4096)",
        "value": round(batch / step_s, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(1e3 * step_s, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (random token ids, random-init weights, synthetic cache contents for the device-timed decode)",
        "impl": "reference",
        "config": {
            "model": "tokenvault preset llama-1b (Llama-3.2-1B shape)", "layers": layers, "hidden": h, "heads": nh, "kv_heads": nkv,
            "head_dim": d, "intermediate": inter, "vocab": v, "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "mean_context": round(mean_ctx, 1), "kv_block_size": 16, "tied_embeddings": cfg.tie_word_embeddings, "rope": "theta 5e5, no llama3 scaling (the reference has none; same bytes and flops)",
            "attention_backend": "gather (its default)", "parallelism": "single-gpu", "package": "unmodified copy of src/tokenvault",
            "peaks": pk["source"],
        },  # fmt: skip
        "e2e": {"value": round(produced / e2e_seconds, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "prefill": {"value": round(PREFILL_TOKENS / p_seconds, 1), "tokens": PREFILL_TOKENS, "ms": round(1e3 * p_seconds, 3),
                    "frac": round(p_flops / p_seconds / (pk["bf16_tflops"] * 1e12), 4)},  # fmt: skip
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--only", choices=["decode", "prefill", "mixed", "attention", "attention-prefill", "gemm", "sample", "load"], help="run one part alone and print a short line (for profiling)")
    ap.add_argument("--preset", default="llama-3.2-1b", help="with --only: the shape (llama-3.2-1b, llama-3.2-3b, llama-3.1-8b)")
    ap.add_argument("--split", type=int, default=0, help="with --only attention: keys per range (0 = the engine's choice)")
    ap.add_argument("--block-size", type=int, default=16, help="with --only attention / attention-prefill: tokens per page")
    ap.add_argument("--temperature", type=float, default=0.8, help="with --only sample (0 = greedy)")
    ap.add_argument("--top-k", type=int, default=50, help="with --only sample (0 = off)")
    ap.add_argument("--top-p", type=float, default=0.9, help="with --only sample (1 = off)")
    ap.add_argument("--short-prompts", action="store_true", help="with --only load: 256 requests with prompts of 16 to 256 tokens and 16 to 128 generated tokens")
    ap.add_argument("--peaked", action="store_true", help="with --only sample: rows with a few likely tokens and a long tail instead of normal noise")
    ap.add_argument("--shape", default="gate_up", help="with --only gemm: qkv, o, gate_up, down or lm_head")
    ap.add_argument("--batch", type=int, default=8, help="with --only decode: the batch")
    ap.add_argument("--context", type=int, default=PROMPT_LEN, help="with --only decode: tokens already in each cache")
    ap.add_argument("--no-graphs", action="store_true", help="with --only: launch kernels one by one instead of replaying a graph")
    args = ap.parse_args()
    if args.gpus > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("bench.py: this engine runs on one GPU; --gpus > 1 is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    if args.only:
        print(json.dumps(run_only(args)))
        return 0
    print(json.dumps(run_own(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
