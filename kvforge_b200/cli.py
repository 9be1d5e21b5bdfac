"""Generate tokens from a model folder or a random-weights preset.

The options that umarhassan-cloud/kvforge's launcher has (scripts/serve.py:41-61) keep their
names and meanings: ``--preset`` / ``--hf-model`` (here a local folder with config.json and
safetensors), ``--device``, ``--dtype``, ``--block-size``, ``--num-blocks``, ``--kv-cache-gb``,
``--max-num-seqs``, ``--max-num-batched-tokens``, ``--max-model-len``.  The sampling options are
the fields of its ``SamplingParams``.  Prompts are token ids (``--prompt-ids "1,2,3"``, one
per use, or ``--prompt-file`` with one comma-separated prompt a line) or, with the byte
tokenizer of the random-weight demos, text (``--prompt``).

    bin/generate --preset tiny-a --prompt-ids 5,17,3 --max-tokens 8 --temperature 0
    bin/generate --hf-model /path/to/Llama-3.2-1B --prompt-ids 128000,9906 --max-tokens 32
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main() -> int:
    from . import PRESETS, ByteTokenizer, CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    src = p.add_mutually_exclusive_group()
    src.add_argument("--preset", choices=sorted(PRESETS), default="tiny-a")
    src.add_argument("--hf-model", "--model", dest="hf_model", help="local folder with config.json and safetensors")
    p.add_argument("--device", default="cuda")
    p.add_argument("--dtype", choices=["float32", "bfloat16"], default="bfloat16")
    p.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--num-blocks", type=int, default=None)
    p.add_argument("--kv-cache-gb", type=float, default=0.25)
    p.add_argument("--max-num-seqs", type=int, default=32)
    p.add_argument("--max-num-batched-tokens", type=int, default=2048)
    p.add_argument("--max-model-len", type=int, default=2048)
    p.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids (repeatable)")
    p.add_argument("--prompt-file", help="file with one comma-separated prompt a line")
    p.add_argument("--prompt", action="append", default=[], help="text, encoded as UTF-8 bytes (random-weight demos)")
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--stats", action="store_true", help="print the engine's figures after the run")
    args = p.parse_args()

    prompts: list = [[int(t) for t in s.split(",") if t.strip()] for s in args.prompt_ids]
    if args.prompt_file:
        for line in Path(args.prompt_file).read_text().splitlines():
            if line.strip():
                prompts.append([int(t) for t in line.split(",") if t.strip()])
    tokenizer = None
    if args.prompt:  # text goes in as bytes, fitted to the vocabulary of the model that will run
        if args.hf_model:
            from .config.model_config import read_config_json

            vocab = int(read_config_json(args.hf_model)["vocab_size"])
        else:
            vocab = PRESETS[args.preset].vocab_size
        tokenizer = ByteTokenizer(vocab)
    prompts.extend(args.prompt)
    if not prompts:
        p.error("give --prompt-ids, --prompt-file or --prompt")

    config = EngineConfig(
        model=None if args.hf_model else PRESETS[args.preset],
        cache=CacheConfig(
            block_size=args.block_size,
            num_blocks=args.num_blocks,
            kv_cache_memory_gb=None if args.num_blocks else args.kv_cache_gb,
        ),
        scheduler=SchedulerConfig(
            max_num_seqs=args.max_num_seqs,
            max_num_batched_tokens=args.max_num_batched_tokens,
            max_model_len=args.max_model_len,
        ),
        device=args.device,
        dtype=args.dtype,
        seed=args.seed,
    )
    engine = InferenceEngine(config, model=args.hf_model, tokenizer=tokenizer)
    kv = engine.kv_cache
    name = args.hf_model or f"kvforge_b200-{args.preset}-random"
    print(f"kvforge_b200: model={name} blocks={kv.num_blocks}x{kv.block_size} kv={kv.memory_bytes / 2**20:.1f} MiB device={args.device}", file=sys.stderr)
    sp = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, ignore_eos=args.ignore_eos)
    for out in engine.generate(prompts, sp):
        print(json.dumps({"request_id": out.request_id, "prompt_token_ids": out.prompt_token_ids, "output_token_ids": out.output_token_ids,
                          "finish_reason": out.finish_reason.value if out.finish_reason else None, "text": out.text}))  # fmt: skip
    if args.stats:
        print(json.dumps(engine.stats(), default=str), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
