"""Replay on the GPU against the plain implementation: the same requests whole, with the
last 32 tokens one by one, in portions of changing size, and mixed with other requests on
so few pages that they are used again; in 32-bit and in bfloat16."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import traces
from helpers import TINY, make_model_dir, random_tokens, rel_err
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"tiny-a": [5, 17, 33, 70, 100], "tiny-b": [1, 9, 40, 71, 130], "tiny-c": [3, 64, 65, 97, 2], "tiny-d": [130, 70, 33, 200, 17], "tiny-e": [66, 140, 9, 35, 101]}
# Error of a logits row: largest difference over the row's largest magnitude.
# float32: the engine's 32-bit kernels against 32-bit torch on the CPU (sums in other orders).
# bfloat16: stored weights are bfloat16 in both, so what differs is the rounding of
# activations (2^-8 each) accumulated over the layers.  Plain bfloat16 arithmetic on these
# tiny models loses 0.7-1.5 % of a row's magnitude on average and up to 5 % at single
# positions; the engine rounds less often (its residual stream and logits are 32-bit).  So a
# row may be off by at most 6 %, and the mean over a trace must not exceed the mean error of
# the plain implementation run in bfloat16 on the same model (``MEAN_SLACK`` for noise).
TOL = {"float32": 2e-5, "bfloat16": 6e-2}
MEAN_SLACK = 1.15


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(tmp, name, store_dtype=torch.bfloat16) for name in TINY}


@pytest.fixture(scope="module")
def oracle(folders):
    """Plain 32-bit logits of every request, whole."""
    out = {}
    for name, d in folders.items():
        vocab = TINY[name]["cfg"].vocab_size
        reqs = {f"{name}-r{i}": random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}
        plain = PlainLlama(d)
        out[name] = (reqs, {rid: plain.logits(t) for rid, t in reqs.items()})
    return out


def plain_bfloat16_mean_error(plain16, reqs, ref) -> float:
    """Mean row error of the plain implementation run in bfloat16."""
    errs = [rel_err(row, ref[rid][i]) for rid, t in reqs.items() for i, row in enumerate(plain16.logits(t))]
    return sum(errs) / len(errs)


@pytest.fixture(scope="module")
def mean_bound(folders, oracle):
    """Per model: the bound on the mean row error of a bfloat16 trace."""
    out = {}
    for name, d in folders.items():
        reqs, ref = oracle[name]
        out[name] = MEAN_SLACK * plain_bfloat16_mean_error(PlainLlama(d, dtype=torch.bfloat16), reqs, ref) + 5e-4
    return out


def run_trace(model_dir, dtype, steps, max_tokens=None, to_host=True, **kw):
    """Replays ``steps``; returns the logits of every step and the runner (for its counters)."""
    from kvforge_b200.replay import TraceRunner

    page = max(64, kw.get("block_size", 16))
    runner = TraceRunner(str(model_dir), dtype, max_tokens or traces.tokens_needed(steps, page), **kw)
    out = []
    for s in steps:
        logits = runner.step(s, to_host=to_host)
        out.append(None if logits is None else logits.clone())
    runner.core.block_manager.check_invariants()
    assert runner.core.block_manager.num_free_blocks == runner.core.block_manager.num_blocks
    return out, runner


def replay_in_process(model_dir, dtype, steps, max_tokens=None, **kw):
    return run_trace(model_dir, dtype, steps, max_tokens, **kw)[0]


def check(steps, outputs, ref_logits, tol, mean_tol=None):
    worst = 0.0
    n = 0
    total = 0.0
    for s, rows, got in zip(steps, traces.wanted_places(steps), outputs):
        if not rows:
            assert got is None
            continue
        assert got.shape[0] == len(rows), f"step {s['step']}: {got.shape[0]} rows for {len(rows)} wanted"
        for i, (rid, pos) in enumerate(rows):
            ref = ref_logits[rid][pos]
            err = rel_err(got[i], ref)
            assert err < tol, f"step {s['step']} request {rid} position {pos}: error {err:.3e} (tolerance {tol})"
            worst = max(worst, err)
            total += err
            n += 1
    assert n > 0
    if mean_tol is not None:
        assert total / n <= mean_tol, f"mean row error {total / n:.3e} exceeds {mean_tol:.3e}"
    return worst


REGIMES = ["whole", "tail", "portions", "mixed"]


def regime_steps(reqs, regime):
    if regime == "whole":
        return traces.whole(reqs)
    if regime == "tail":
        return traces.tail_one_by_one(reqs, 32)
    if regime == "portions":
        return traces.portions(reqs)
    prompt_lens = {rid: max(1, len(t) - 12) for rid, t in reqs.items()}
    steps = traces.mixed(reqs, prompt_lens, max_live=4, seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len(e["tokens"]) == 1 for s in steps for e in s["entries"]) and any(len(e["tokens"]) > 1 for s in steps for e in s["entries"])
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("regime", REGIMES)
def test_replay_regimes(folders, oracle, mean_bound, name, dtype, regime):
    reqs, ref = oracle[name]
    steps = regime_steps(reqs, regime)
    outputs = replay_in_process(folders[name], dtype, steps)
    check(steps, outputs, ref, TOL[dtype], mean_bound[name] if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", [n for n in TINY if TINY[n]["block_size"] != 16])
@pytest.mark.parametrize("regime", REGIMES)
def test_replay_regimes_at_the_models_own_page_size(folders, oracle, mean_bound, name, dtype, regime):
    """Pages of 8 (tiny-b), 4 (tiny-c) and 32 (tiny-e) tokens instead of the replay program's 16."""
    reqs, ref = oracle[name]
    steps = regime_steps(reqs, regime)
    outputs = replay_in_process(folders[name], dtype, steps, block_size=TINY[name]["block_size"])
    check(steps, outputs, ref, TOL[dtype], mean_bound[name] if dtype == "bfloat16" else None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("regime", REGIMES)
def test_replay_regimes_as_captured_graphs(folders, oracle, name, dtype, regime):
    """The same four cuttings the way bfloat16 generation runs them by default: steps of single
    tokens and steps of more than 16 tokens replayed as CUDA graphs made for padded shapes
    (tokens up to a multiple of 64, sequences up to a bucket), every shape captured the first
    time it comes.  A step asks for the last row of each entry, since a step that wants more rows
    than it has sequences is not replayed as a graph."""
    reqs, ref = oracle[name]
    steps = traces.last_only(regime_steps(reqs, regime))
    outputs, runner = run_trace(folders[name], dtype, steps, block_size=TINY[name]["block_size"], cuda_graphs=True)
    check(steps, outputs, ref, TOL[dtype])
    mr = runner.core.runner
    forms = {key[4] for key in mr._graphs}
    if regime != "whole":
        assert True in forms, "no step of single tokens was replayed as a graph"
    if any(sum(len(e["tokens"]) for e in s["entries"]) >= 17 for s in steps):
        assert False in forms, "no step of many tokens was replayed as a graph"
    assert mr.num_graph_kernels > 0


DECODER_MODELS = ["tiny-b", "tiny-d", "tiny-e"]


@pytest.fixture(scope="module")
def decoder_oracle(folders):
    """Per model and number of live requests: requests of different lengths and their plain logits."""
    cache = {}

    def get(name, live):
        if (name, live) not in cache:
            import random

            rng = random.Random(live)
            vocab = TINY[name]["cfg"].vocab_size
            reqs = {f"{name}-m{i}": random_tokens(vocab, rng.randint(14, 40), seed=500 + i) for i in range(live + live // 2)}
            prompt_lens = {rid: max(1, len(t) - rng.randint(6, 12)) for rid, t in reqs.items()}
            plain = PlainLlama(folders[name])
            cache[(name, live)] = (reqs, prompt_lens, {rid: plain.logits(t) for rid, t in reqs.items()})
        return cache[(name, live)]

    return get


@pytest.mark.parametrize("mode", ["float32", "bfloat16", "bfloat16-graphs"])
@pytest.mark.parametrize("name", DECODER_MODELS)
@pytest.mark.parametrize("live", [17, 24, 33, 64])
def test_many_requests_decoding_at_once(folders, decoder_oracle, name, mode, live):
    """Steps of 17 to 64 single decoded tokens, with requests leaving and joining: above 16 rows
    every matrix product of a bfloat16 step takes another route than below (the library instead of
    the decode GEMM, its product over slices of K for the narrow outputs), the graphs are those of
    the buckets 32 and 64, and a joining prompt makes a mixed step with dozens of single tokens."""
    reqs, prompt_lens, ref = decoder_oracle(name, live)
    steps = traces.many_decoders(reqs, prompt_lens, live, seed=live)
    assert any(len(s["entries"]) == live and all(len(e["tokens"]) == 1 for e in s["entries"]) for s in steps)
    dtype = mode.split("-")[0]
    outputs, runner = run_trace(folders[name], dtype, steps, max_live=64, block_size=TINY[name]["block_size"], cuda_graphs=mode.endswith("graphs"))
    check(steps, outputs, ref, TOL[dtype])
    if mode.endswith("graphs"):
        buckets = {key[1] for key in runner.core.runner._graphs if key[4]}
        assert (64 if live > 32 else 32) in buckets


def test_float32_logits_of_a_request_do_not_depend_on_how_many_decode_beside_it(folders):
    """One request with a context of several hundred keys decodes alone and beside 129 others
    (260 pairs of sequence and kv head).  In 32-bit the key ranges of the decode attention have one
    size whatever the batch, and every product sums in a fixed order, so the rows are bit-equal."""
    name = "tiny-a"
    vocab = TINY[name]["cfg"].vocab_size
    long = random_tokens(vocab, 604, seed=77)
    others = {f"o{i}": random_tokens(vocab, 6, seed=900 + i) for i in range(129)}
    alone = traces.tail_one_by_one({"x": long}, tail=4)
    crowd = [{"step": 0, "entries": [{"id": "x", "tokens": long[:600], "want": [599]}], "end": []}]
    for i in range(0, 129, 43):  # the short prompts, 43 a step, all but their last token
        crowd.append({"step": len(crowd), "entries": [{"id": rid, "tokens": t[:5], "want": [4]} for rid, t in list(others.items())[i : i + 43]], "end": []})
    for k in range(4):
        entries = [{"id": "x", "tokens": [long[600 + k]], "want": [0]}]
        if k == 0:
            entries += [{"id": rid, "tokens": [t[5]], "want": [0]} for rid, t in others.items()]
        crowd.append({"step": len(crowd), "entries": entries, "end": list(others) if k == 0 else (["x"] if k == 3 else [])})
    a = replay_in_process(folders[name], "float32", alone, max_live=130)
    b = replay_in_process(folders[name], "float32", crowd, max_live=130)
    assert torch.equal(a[0][0], b[0][0])  # the prompt's last row
    for k in range(4):
        assert torch.equal(a[1 + k][0], b[4 + k][0]), f"decoded token {k}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_changes_nothing_beyond_rounding(folders, oracle, dtype):
    """The same positions through three cuttings agree with each other far more closely than
    the storage type's tolerance against the oracle."""
    name = "tiny-b"
    reqs, _ = oracle[name]
    got = {}
    for regime, steps in (("whole", traces.whole(reqs)), ("portions", traces.portions(reqs)), ("tail", traces.tail_one_by_one(reqs, 32))):
        outs = replay_in_process(folders[name], dtype, steps)
        for rows, g in zip(traces.wanted_places(steps), outs):
            for i, key in enumerate(rows):
                got.setdefault(key, {})[regime] = g[i]
    bound = 1e-5 if dtype == "float32" else 2e-2
    for key, by in got.items():
        for regime in ("portions", "tail"):
            if regime in by:
                assert rel_err(by[regime], by["whole"]) < bound, (key, regime)


def test_bfloat16_engine_is_no_worse_than_plain_bfloat16(folders, oracle):
    """The engine's bfloat16 error against 32-bit stays within that of a plain bfloat16 run
    (which rounds more often: the engine keeps the residual stream in 32-bit)."""
    name = "tiny-a"
    reqs, ref = oracle[name]
    plain16 = PlainLlama(folders[name], dtype=torch.bfloat16)
    steps = traces.whole(reqs)
    outputs = replay_in_process(folders[name], "bfloat16", steps)
    for rows, got in zip(traces.wanted_places(steps), outputs):
        rid = rows[0][0]
        p16 = plain16.logits(reqs[rid])
        e_plain = sum(rel_err(p16[i], ref[rid][i]) for i in range(len(reqs[rid]))) / len(reqs[rid])
        e_engine = sum(rel_err(got[i], ref[rid][i]) for i in range(len(reqs[rid]))) / len(reqs[rid])
        if len(reqs[rid]) >= 30:  # a mean over few rows is noise
            assert e_engine <= MEAN_SLACK * e_plain + 5e-4, (rid, e_engine, e_plain)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """Two hundred tokens decoded one by one after a short prompt (tiny-b: llama3 scaling,
    positions well past the original context of 64)."""
    name = "tiny-b"
    toks = random_tokens(TINY[name]["cfg"].vocab_size, 230, seed=9)
    ref = {"long": PlainLlama(folders[name]).logits(toks)}
    steps = traces.tail_one_by_one({"long": toks}, tail=222)
    outputs = replay_in_process(folders[name], dtype, steps)
    check(steps, outputs, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_first_tokens_of_a_sequence(folders, name, dtype):
    toks = random_tokens(TINY[name]["cfg"].vocab_size, 4, seed=3)
    ref = {"s": PlainLlama(folders[name]).logits(toks)}
    steps = [{"step": i, "entries": [{"id": "s", "tokens": [t], "want": [0]}], "end": ["s"] if i == 3 else []} for i, t in enumerate(toks)]
    check(steps, replay_in_process(folders[name], dtype, steps), ref, TOL[dtype])


def test_pages_are_used_again_without_leaking_old_contents(folders, oracle):
    """A pool of exactly one request's size: every request gets the pages of the one before."""
    name = "tiny-a"
    reqs, ref = oracle[name]
    steps = traces.portions(reqs)
    outputs = replay_in_process(folders[name], "float32", steps, max_tokens=128)
    check(steps, outputs, ref, TOL["float32"])


def test_trace_run_program(folders, oracle, tmp_path):
    """The program itself: standard input, ``done <step>`` lines, little-endian files."""
    name = "tiny-a"
    reqs, ref = oracle[name]
    prompt_lens = {rid: max(1, len(t) - 8) for rid, t in reqs.items()}
    steps = traces.mixed(reqs, prompt_lens, max_live=4, seed=2)
    steps.insert(3, {"step": 1000, "entries": [], "end": []})
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders[name]), "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(traces.tokens_needed(steps))],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600,
    )  # fmt: skip
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = TINY[name]["cfg"].vocab_size
    outputs = []
    for s, rows in zip(steps, traces.wanted_places(steps)):
        f = out / f"{s['step']}.f32"
        if not rows:
            assert not f.exists()
            outputs.append(None)
            continue
        a = np.fromfile(f, dtype="<f4")
        assert a.size == len(rows) * vocab
        outputs.append(torch.from_numpy(a.reshape(len(rows), vocab)))
    check(steps, outputs, ref, TOL["float32"])


def test_a_preset_with_a_seed_stands_for_a_model_folder(tmp_path):
    """``--preset NAME --seed S`` makes on the device the weights that the random-weights mode
    writes into a folder for the same shape and seed (drawn on the same device): same logits."""
    from kvforge_b200 import PRESETS
    from kvforge_b200.models.folder import write_random_model
    from kvforge_b200.replay import TraceRunner

    folder = write_random_model(tmp_path / "m", PRESETS["tiny-b"], seed=4, store_dtype=torch.float32, device="cuda")
    toks = random_tokens(PRESETS["tiny-b"].vocab_size, 40, seed=8)
    steps = traces.portions({"a": toks})
    a = run_trace(folder, "float32", steps)[0]
    runner = TraceRunner(None, "float32", traces.tokens_needed(steps), preset="tiny-b", seed=4)
    b = [runner.step(s) for s in steps]
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    other = TraceRunner(None, "float32", traces.tokens_needed(steps), preset="tiny-b", seed=5)
    assert not torch.equal(other.step(steps[0]), a[0])
    with pytest.raises(ValueError):
        TraceRunner(None, "float32", 64)
