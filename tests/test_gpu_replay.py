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


def replay_in_process(model_dir, dtype, steps, max_tokens=None):
    from kvforge_b200.replay import TraceRunner

    runner = TraceRunner(str(model_dir), dtype, max_tokens or traces.tokens_needed(steps))
    out = []
    for s in steps:
        logits = runner.step(s)
        out.append(None if logits is None else logits.clone())
    runner.core.block_manager.check_invariants()
    assert runner.core.block_manager.num_free_blocks == runner.core.block_manager.num_blocks
    return out


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("regime", ["whole", "tail", "portions", "mixed"])
def test_replay_regimes(folders, oracle, mean_bound, name, dtype, regime):
    reqs, ref = oracle[name]
    if regime == "whole":
        steps = traces.whole(reqs)
    elif regime == "tail":
        steps = traces.tail_one_by_one(reqs, 32)
    elif regime == "portions":
        steps = traces.portions(reqs)
    else:
        prompt_lens = {rid: max(1, len(t) - 12) for rid, t in reqs.items()}
        steps = traces.mixed(reqs, prompt_lens, max_live=4, seed=5)
        assert max(len(s["entries"]) for s in steps) >= 3
        assert any(len(e["tokens"]) == 1 for s in steps for e in s["entries"]) and any(len(e["tokens"]) > 1 for s in steps for e in s["entries"])
    outputs = replay_in_process(folders[name], dtype, steps)
    check(steps, outputs, ref, TOL[dtype], mean_bound[name] if dtype == "bfloat16" else None)


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
