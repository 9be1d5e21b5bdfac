"""Contexts of ten thousand tokens and more through the engine, against the plain implementation:
a prompt of 12,300 tokens whole, prompts in portions of thousands of tokens beside decoded tokens
with a long reach, and four requests decoding together (16 (sequence, kv head) pairs of more than
ten thousand keys each: the decode kernel widens its ranges of keys), in 32-bit and in bfloat16,
eager and as captured graphs.  The queries and keys of this model are scaled up so that a
position's attention rests on few keys spread over the whole context: a range of keys that was
skipped, or read from another request's page, moves the logits."""

from __future__ import annotations

import json

import pytest
import torch

import traces
from helpers import random_tokens, rel_err
from kvforge_b200 import ModelConfig, RopeScaling
from kvforge_b200.models.folder import write_random_model
from kvforge_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

CFG = ModelConfig(
    vocab_size=331, hidden_size=256, num_layers=2, num_heads=8, num_kv_heads=4, head_dim=64, intermediate_size=416,
    rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=RopeScaling(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=2048),
    tie_word_embeddings=True, max_position_embeddings=16384,
)  # fmt: skip
PROMPTS = {"a": 12300, "b": 9800, "c": 2100, "d": 11111}
TAILS = {"a": 16, "b": 11, "c": 10, "d": 7}
SHARPER = 2.0  # factor on the query and key projections


@pytest.fixture(scope="module")
def long_model(tmp_path_factory):
    folder = tmp_path_factory.mktemp("long") / "head-64-16k"
    write_random_model(folder, CFG, seed=9, store_dtype=torch.bfloat16, init_std=0.06, norm_std=0.05)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {}
    for name in f.keys():
        t = f.tensor(name).clone()
        if name.endswith(("q_proj.weight", "k_proj.weight")):
            t = (t.float() * SHARPER).to(t.dtype)
        tensors[name] = t
    f.close()
    write_safetensors(folder / "model.safetensors", tensors)
    assert json.loads((folder / "config.json").read_text())["max_position_embeddings"] == 16384
    reqs = {rid: random_tokens(CFG.vocab_size, n + TAILS[rid], seed=20 + i) for i, (rid, n) in enumerate(PROMPTS.items())}
    steps = traces.staggered(reqs, PROMPTS, sizes=(12300, 3000, 4096, 2048, 1024))
    assert len(steps[0]["entries"][0]["tokens"]) == 12300
    assert sum(1 for s in steps if len(s["entries"]) == 4 and all(len(e["tokens"]) == 1 for e in s["entries"])) >= 4
    assert any(len(s["entries"]) >= 3 and max(len(e["tokens"]) for e in s["entries"]) > 2000 for s in steps)
    wanted = {}
    for rows in traces.wanted_places(steps):
        for rid, pos in rows:
            wanted.setdefault(rid, set()).add(pos)
    torch.backends.cuda.matmul.allow_tf32 = False
    ref, err16 = {}, []
    for dtype in (torch.float32, torch.bfloat16):
        plain = PlainLlama(folder, dtype=dtype, device="cuda")
        for rid, toks in reqs.items():
            rows = plain.logits(toks).float().cpu()
            if dtype == torch.float32:
                ref[rid] = {p: rows[p].clone() for p in wanted[rid]}
            else:
                err16 += [rel_err(rows[p], ref[rid][p]) for p in wanted[rid]]
            del rows
        del plain
        torch.cuda.empty_cache()
    return folder, steps, ref, sum(err16) / len(err16)


@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("float32", True), ("bfloat16", False), ("bfloat16", True)])
def test_long_contexts_whole_in_portions_and_decoding_together(long_model, dtype, graphs):
    from test_gpu_replay import MEAN_SLACK, TOL, check, run_trace

    folder, steps, ref, plain16 = long_model
    outputs, runner = run_trace(folder, dtype, steps, max_live=4, cuda_graphs=graphs)
    if graphs:
        assert runner.core.runner.num_graph_kernels > 0
    check(steps, outputs, ref, TOL[dtype], MEAN_SLACK * plain16 + 5e-4 if dtype == "bfloat16" else None)
