"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
``EngineCore`` (the model, step function, page allocator and kernels that generation uses).
The nearest thing in umarhassan-cloud/kvforge is the test that drives ``ModelRunner.execute``
with explicit batch items (tests/test_paged_attention.py:93-113).

Input, one JSON object a line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits are
wanted.  All entries of a step run as one batch.  ``end``: requests that are finished after
the step; their pages are given back.  A step with wanted places writes
``<out>/<step>.f32``: little-endian float32 ``[wanted, vocab]`` in the order of the entries
and of ``want``.  After every step ``done <step>`` is printed and flushed.

``--preset NAME --seed S`` stands for ``--model``: the named shape with random weights made
on the device.  The page size is 16 tokens unless ``--block-size`` says otherwise, the pool holds
``--max-tokens`` tokens (each request rounded up to 64, or to the page if that is larger)
unless ``--num-blocks`` gives it in pages, and ``--cuda-graphs`` replays the steps the way
bfloat16 generation does by default: captured graphs for padded shapes, every shape captured
the first time it comes.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE = 16  # tokens per page of the replay engine unless --block-size is given
ROUND = 64  # --max-tokens counts each request rounded up to this (or to the page, if larger)


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--preset", help="a named shape instead of a folder: random weights made on the device from --seed")
    ap.add_argument("--seed", type=int, default=0, help="with --preset: seed of the random weights")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    ap.add_argument("--max-live", type=int, default=16, help="most requests live at a time")
    ap.add_argument("--block-size", type=int, default=PAGE, help="tokens per page of the cache")
    ap.add_argument("--num-blocks", type=int, default=None, help="pages of the pool (default: what --max-tokens needs)")
    ap.add_argument("--cuda-graphs", action="store_true", help="replay steps as captured CUDA graphs, as generation does")
    return ap.parse_args(argv)


def pages_for(max_tokens: int, block_size: int, max_live: int) -> int:
    """Pages that hold ``max_tokens`` tokens when each live request's count was rounded up to
    ``ROUND``: with pages that divide ``ROUND`` exactly that many tokens; with other page sizes
    every live request may waste the better part of a page on top."""
    pages = -(-int(max_tokens) // block_size)
    if ROUND % block_size:
        pages += max_live
    return max(1, pages)


class TraceRunner:
    def __init__(
        self,
        model_dir: str | None,
        dtype: str,
        max_tokens: int,
        max_live: int = 16,
        block_size: int = PAGE,
        num_blocks: int | None = None,
        cuda_graphs: bool = False,
        preset: str | None = None,
        seed: int = 0,
    ) -> None:
        from .config.engine_config import CacheConfig
        from .engine.core import EngineCore, spec_from_config

        block_size = int(block_size)
        if block_size <= 0:
            raise ValueError("--block-size must be positive")
        if num_blocks is None:
            num_blocks = pages_for(max_tokens, block_size, max_live)
        budget = max(int(max_tokens), block_size)
        if (model_dir is None) == (preset is None):
            raise ValueError("give a model folder or a preset, not both")
        if preset is not None:
            from .config.registry import PRESETS

            if preset not in PRESETS:
                raise ValueError(f"no preset named {preset!r} (known: {sorted(PRESETS)})")
            make = lambda **kw: EngineCore(spec_from_config(PRESETS[preset]), seed=seed, **kw)  # noqa: E731
        else:
            make = lambda **kw: EngineCore.from_model_dir(model_dir, **kw)  # noqa: E731
        self.core = make(
            dtype=dtype,
            cache=CacheConfig(block_size=block_size, num_blocks=int(num_blocks), watermark=0.0),
            max_num_seqs=max_live,
            max_num_batched_tokens=budget,
            max_model_len=budget,
            cuda_graphs=bool(cuda_graphs),
            # captured graphs hold buffer addresses, so buffers are made for the whole budget at once
            lazy_buffers=not cuda_graphs,
        )
        self.core.runner.graph_after = 1  # a replayed trace shows each shape once: capture it the first time
        self.lengths: dict[str, int] = {}

    def step(self, record: dict, to_host: bool = True):
        """Runs one step; returns the float logits ``[wanted, vocab]`` on the host (or, with
        ``to_host=False``, a copy on the device), or ``None`` if nothing was wanted."""
        from .engine.step import BatchItem

        core = self.core
        bm, slots = core.block_manager, core.state_slots
        vocab = core.spec.vocab_size
        items = []
        for e in record.get("entries", []):
            rid, tokens = str(e["id"]), [int(t) for t in e["tokens"]]
            if not tokens:
                continue
            if any(t < 0 or t >= vocab for t in tokens):
                raise ValueError(f"step {record.get('step')}: request {rid} has a token id outside the vocabulary of {vocab}")
            start = self.lengths.get(rid, 0)
            total = start + len(tokens)
            if rid not in self.lengths:
                bm.allocate(rid, total, len(tokens))
                slots.allocate(rid)
            else:
                bm.append_slots(rid, total, start)
            self.lengths[rid] = total
            items.append(BatchItem(rid, tokens, start, [int(i) for i in e.get("want", [])]))
        logits = core.runner.step(items) if items else None
        host = None
        if logits is not None and logits.shape[0] > 0:
            host = logits.cpu() if to_host else logits.clone()
        elif logits is not None:
            import torch

            torch.cuda.current_stream().synchronize()
        if items:
            core.rt.check_error_flag()
        for rid in record.get("end", []):
            rid = str(rid)
            bm.free(rid)
            slots.free(rid)
            self.lengths.pop(rid, None)
        return host


def main(argv=None) -> int:
    args = parse_args(argv)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    runner = TraceRunner(args.model, args.dtype, args.max_tokens, args.max_live, args.block_size, args.num_blocks, args.cuda_graphs, args.preset, args.seed)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = runner.step(record)
        if logits is not None:
            logits.numpy().astype("<f4", copy=False).tofile(out / f"{step}.f32")
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
