"""Generation through the Python entry point against greedy decoding by full recomputation
with the plain implementation; what the scheduler does under pressure must not change a token."""

from __future__ import annotations

import random

import pytest
import torch

from helpers import TINY, make_model_dir, random_tokens
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(tmp, name, store_dtype=torch.bfloat16) for name in TINY}


def engine_for(folder, name, dtype="float32", num_blocks=256, **sched):
    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, SchedulerConfig

    sched.setdefault("max_num_seqs", 8)
    sched.setdefault("max_num_batched_tokens", 256)
    sched.setdefault("max_model_len", 256)
    cuda_graphs = sched.pop("cuda_graphs", True)
    async_output = sched.pop("async_output", True)
    cfg = EngineConfig(
        cache=CacheConfig(block_size=TINY[name]["block_size"], num_blocks=num_blocks),
        scheduler=SchedulerConfig(**sched),
        dtype=dtype,
        cuda_graphs=cuda_graphs,
        async_output=async_output,
    )
    return InferenceEngine(cfg, model=folder)


def greedy(n):
    from kvforge_b200 import SamplingParams

    return SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True)


def prompts_for(name, lengths, seed=0):
    vocab = TINY[name]["cfg"].vocab_size
    return [random_tokens(vocab, n, seed=seed + i) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("name", list(TINY))
def test_batched_greedy_generation_equals_plain(folders, name):
    prompts = prompts_for(name, [2, 30, 7, 19, 1, 12])
    plain = PlainLlama(folders[name])
    engine = engine_for(folders[name], name)
    outs = engine.generate(prompts, greedy(10))
    assert [o.prompt_token_ids for o in outs] == prompts
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy(p, 10)
        assert o.finished and o.finish_reason.value == "length"
    assert engine.block_manager.num_free_blocks == engine.block_manager.num_blocks
    engine.block_manager.check_invariants()


@pytest.mark.parametrize("name", ["tiny-a", "tiny-d", "tiny-e"])
def test_bfloat16_generation_with_and_without_graphs(folders, name):
    """The bfloat16 path generates the same tokens whether single-token steps are replayed
    as CUDA graphs or launched one kernel at a time, and they are the plain model's tokens
    wherever its top-2 margin is larger than bfloat16 rounding."""
    prompts = prompts_for(name, [5, 17, 33, 9], seed=40)
    a = engine_for(folders[name], name, "bfloat16", cuda_graphs=True).generate(prompts, greedy(12))
    b = engine_for(folders[name], name, "bfloat16", cuda_graphs=False).generate(prompts, greedy(12))
    assert [o.output_token_ids for o in a] == [o.output_token_ids for o in b]
    plain = PlainLlama(folders[name])
    checked = 0
    for p, o in zip(prompts, a):
        ids = list(p)
        for tok in o.output_token_ids:
            logits = plain.logits(ids)[-1]
            top = logits.topk(2).values
            if float(top[0] - top[1]) > 0.08 * float(logits.abs().max()):
                assert tok == int(logits.argmax())
                checked += 1
            ids.append(tok)
    assert checked >= 24, f"only {checked} of 48 tokens had a margin wide enough to compare"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_dozens_of_decoding_requests_beside_short_prompts_that_arrive_late(folders, dtype):
    """About forty requests decode while short prompts keep arriving, with room for 64 sequences:
    such a step holds 33 to 63 single tokens and a portion of a few tokens, at most 64 tokens in
    all, so as a graph it is padded to 64 tokens in 64 sequences, the very numbers of the graph of
    64 decoding requests.  The two are different graphs; taking one for the other would compute
    only the last query of the portion.  Tokens are the plain model's: all of them in 32-bit, in
    bfloat16 wherever its top-2 margin is larger than bfloat16 rounding."""
    name = "tiny-d"
    rng = random.Random(3)
    prompts = prompts_for(name, [rng.randint(5, 20) for _ in range(58)], seed=70)
    lengths = [rng.randint(10, 22) for _ in prompts]
    plain = PlainLlama(folders[name])
    engine = engine_for(folders[name], name, dtype, num_blocks=400, max_num_seqs=64, max_num_batched_tokens=256, max_model_len=64)
    ids = [engine.add_request(p, greedy(n)) for p, n in zip(prompts[:40], lengths[:40])]
    late = list(zip(prompts[40:], lengths[40:]))
    done = {}
    while engine.has_unfinished_requests():
        if late and engine.runner.num_forward_passes >= 2 and engine.runner.num_forward_passes % 2 == 0:
            p, n = late.pop(0)  # one more prompt with every other step; the steps between hold decoding requests alone
            ids.append(engine.add_request(p, greedy(n)))
        for out in engine.step():
            if out.finished:
                done[out.request_id] = out
    shapes = set(engine.runner._graphs)
    assert any(k[:2] == (64, 64) and k[4] for k in shapes) and any(k[:2] == (64, 64) and not k[4] for k in shapes), sorted(shapes)
    assert any(not k[4] and k[3] for k in shapes), "no mixed step was replayed as a graph"
    engine.core.rt.check_error_flag()
    checked = 0
    for rid, p, n in zip(ids, prompts, lengths):
        got = done[rid].output_token_ids
        assert len(got) == n
        if dtype == "float32":
            assert got == plain.greedy(p, n), rid
            checked += n
            continue
        seq = list(p)
        for tok in got:
            logits = plain.logits(seq)[-1]
            top = logits.topk(2).values
            if float(top[0] - top[1]) > 0.08 * float(logits.abs().max()):
                assert tok == int(logits.argmax()), rid
                checked += 1
            seq.append(tok)
    assert checked > 300
    assert engine.block_manager.num_free_blocks == engine.block_manager.num_blocks


def test_requests_that_join_late_and_leave_early(folders):
    name = "tiny-b"
    prompts = prompts_for(name, [9, 40, 5, 21], seed=7)
    plain = PlainLlama(folders[name])
    engine = engine_for(folders[name], name, max_prefill_chunk=16)
    ids = [engine.add_request(prompts[0], greedy(12)), engine.add_request(prompts[1], greedy(3))]
    done = {}
    step = 0
    while engine.has_unfinished_requests():
        if step == 3:
            ids.append(engine.add_request(prompts[2], greedy(8)))
        if step == 5:
            ids.append(engine.add_request(prompts[3], greedy(6)))
        for out in engine.step():
            if out.finished:
                done[out.request_id] = out
        step += 1
    for rid, p, n in zip(ids, prompts, [12, 3, 8, 6]):
        assert done[rid].output_token_ids == plain.greedy(p, n)
    assert engine.block_manager.num_free_blocks == engine.block_manager.num_blocks


def test_chunked_prefill_changes_no_token(folders):
    name = "tiny-a"
    prompts = prompts_for(name, [59, 40], seed=3)
    plain = PlainLlama(folders[name])
    engine = engine_for(folders[name], name, max_num_batched_tokens=16, max_model_len=128)
    outs = engine.generate(prompts, greedy(8))
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy(p, 8)
    assert engine.runner.num_forward_passes > 8 + 4


def test_when_pages_run_out_requests_are_preempted_and_tokens_do_not_change(folders):
    name = "tiny-c"  # pages of 4
    prompts = prompts_for(name, [10, 14, 9, 12, 11, 13], seed=11)
    plain = PlainLlama(folders[name])
    engine = engine_for(folders[name], name, num_blocks=14, max_num_seqs=6)
    outs = engine.generate(prompts, greedy(10))
    assert engine.scheduler.num_preemptions > 0
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy(p, 10)
    engine.block_manager.check_invariants()
    assert engine.block_manager.num_free_blocks == 14


def test_preemption_in_bfloat16_with_graphs_and_mixed_steps(folders):
    """Pages run out in the bfloat16 engine (tensor-core kernels, graphs, tokens read a step
    late): requests are preempted and run again as portions beside decoding ones; every request
    finishes, no page is lost, and the tokens are the plain model's wherever its top-2 margin is
    larger than bfloat16 rounding."""
    name = "tiny-d"  # pages of 16
    prompts = prompts_for(name, [40, 55, 33, 61, 47, 52], seed=21)
    engine = engine_for(folders[name], name, "bfloat16", num_blocks=22, max_num_seqs=6, max_num_batched_tokens=96, max_model_len=160)
    outs = engine.generate(prompts, greedy(40))
    assert engine.scheduler.num_preemptions > 0
    engine.core.rt.check_error_flag()
    engine.block_manager.check_invariants()
    assert engine.block_manager.num_free_blocks == 22
    plain = PlainLlama(folders[name])
    checked = 0
    for p, o in zip(prompts, outs):
        assert o.finished and len(o.output_token_ids) == 40
        ids = list(p)
        for tok in o.output_token_ids:
            logits = plain.logits(ids)[-1]
            top = logits.topk(2).values
            if float(top[0] - top[1]) > 0.08 * float(logits.abs().max()):
                assert tok == int(logits.argmax())
                checked += 1
            else:
                break  # past a close call the two may follow different tokens
            ids.append(tok)
    assert checked > 20


def test_stop_token_abort_and_length_limit(folders):
    from kvforge_b200 import SamplingParams

    name = "tiny-a"
    plain = PlainLlama(folders[name])
    prompt = prompts_for(name, [6], seed=1)[0]
    want = plain.greedy(prompt, 8)
    engine = engine_for(folders[name], name)
    out = engine.generate([prompt], SamplingParams(max_tokens=8, temperature=0.0, stop_token_ids=[want[3]]))[0]
    assert out.output_token_ids == want[: want.index(want[3]) + 1] and out.finish_reason.value == "stop"
    # the model's length limit ends a request
    engine = engine_for(folders[name], name, max_model_len=12)
    out = engine.generate([prompt], greedy(50))[0]
    assert len(out.output_token_ids) == 6 and out.finish_reason.value == "length"
    # abort gives the pages back
    rid = engine.add_request(prompt, greedy(5))
    engine.step()
    assert engine.block_manager.num_free_blocks < engine.block_manager.num_blocks
    assert engine.abort_request(rid) and not engine.has_unfinished_requests()
    assert engine.block_manager.num_free_blocks == engine.block_manager.num_blocks
    with pytest.raises(ValueError):
        engine.add_request([0, 256], greedy(1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_reading_tokens_a_step_late_changes_no_output(folders, dtype):
    """Tokens read while the next step runs (the default) and tokens read before it: the same
    outputs, also when stop tokens end requests at different times and pages are short."""
    from kvforge_b200 import SamplingParams

    name = "tiny-c"
    prompts = prompts_for(name, [10, 14, 9, 12, 3, 13], seed=31)
    plain = PlainLlama(folders[name])
    stops = [plain.greedy(p, 9)[5] for p in prompts]  # each request stops at a token it will really produce
    sp = [SamplingParams(max_tokens=11, temperature=0.0, stop_token_ids=[t]) for t in stops]
    runs = {}
    for mode in (True, False):
        engine = engine_for(folders[name], name, dtype, num_blocks=16, max_num_seqs=6, async_output=mode)
        outs = engine.generate(prompts, sp)
        runs[mode] = [(o.output_token_ids, o.finish_reason.value) for o in outs]
        assert engine.block_manager.num_free_blocks == 16 and not engine.has_unfinished_requests()
        engine.block_manager.check_invariants()
    assert runs[True] == runs[False]
    if dtype == "float32":
        for p, t, (ids, reason) in zip(prompts, stops, runs[True]):
            want = plain.greedy(p, 11)
            want = want[: want.index(t) + 1]
            assert ids == want and reason == "stop"


def test_temperature_sampling_does_not_depend_on_the_batch(folders):
    """Every request draws from its own stream: the tokens of a request are the same alone,
    in a batch, and under chunked prefill."""
    from kvforge_b200 import SamplingParams

    name = "tiny-b"
    prompts = prompts_for(name, [1, 9, 40, 71], seed=23)
    sp = [SamplingParams(max_tokens=12, temperature=0.8, ignore_eos=True, seed=100 + i) for i in range(4)]
    batch = engine_for(folders[name], name).generate(prompts, sp)
    chunked = engine_for(folders[name], name, max_prefill_chunk=16, max_num_batched_tokens=32).generate(prompts, sp)
    alone = [engine_for(folders[name], name).generate([p], [s])[0] for p, s in zip(prompts[:2], sp[:2])]
    assert [o.output_token_ids for o in batch] == [o.output_token_ids for o in chunked]
    assert [o.output_token_ids for o in batch[:2]] == [o.output_token_ids for o in alone]
    assert len({tuple(o.output_token_ids) for o in batch}) > 1
    other = engine_for(folders[name], name).generate(prompts[2:3], [SamplingParams(max_tokens=12, temperature=0.8, ignore_eos=True, seed=999)])
    assert other[0].output_token_ids != batch[2].output_token_ids


def test_top_k_one_is_greedy(folders):
    from kvforge_b200 import SamplingParams

    name = "tiny-a"
    prompt = prompts_for(name, [11], seed=2)[0]
    plain = PlainLlama(folders[name])
    out = engine_for(folders[name], name).generate([prompt], SamplingParams(max_tokens=6, temperature=1.5, top_k=1, ignore_eos=True))[0]
    assert out.output_token_ids == plain.greedy(prompt, 6)


def test_random_weights_mode_needs_no_folder():
    from kvforge_b200 import PRESETS, CacheConfig, EngineConfig, InferenceEngine, SchedulerConfig

    cfg = EngineConfig(model=PRESETS["tiny-b"], cache=CacheConfig(block_size=8, num_blocks=64),
                       scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64), dtype="bfloat16", seed=5)  # fmt: skip
    a = InferenceEngine(cfg).generate([[1, 2, 3]], greedy(5))[0].output_token_ids
    b = InferenceEngine(cfg).generate([[1, 2, 3]], greedy(5))[0].output_token_ids
    assert a == b and len(a) == 5
    stats = InferenceEngine(cfg).stats()
    assert stats["kv_cache"]["num_free_blocks"] == 64


def test_the_command_line_generates_the_plain_models_tokens(folders):
    """bin/generate on a model folder, greedy, float32: the tokens of the plain implementation."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    name = "tiny-b"
    prompts = prompts_for(name, [9, 3], seed=70)
    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, str(root / "bin" / "generate"), "--hf-model", str(folders[name]), "--dtype", "float32", "--block-size", "8",
           "--num-blocks", "64", "--max-model-len", "128", "--max-num-batched-tokens", "64", "--max-tokens", "6", "--temperature", "0", "--ignore-eos"]  # fmt: skip
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    outs = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    plain = PlainLlama(folders[name])
    assert [o["prompt_token_ids"] for o in outs] == prompts
    for p, o in zip(prompts, outs):
        assert o["output_token_ids"] == plain.greedy(p, 6) and o["finish_reason"] == "length"


def test_the_command_line_takes_text_with_the_default_preset():
    """``bin/generate --prompt "text"`` with the default preset (a vocabulary of 256 entries: no
    room for marks beside the bytes): the prompt is the text's bytes, and tokens come out."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, str(root / "bin" / "generate"), "--prompt", "hello", "--prompt", "page", "--max-tokens", "5", "--temperature", "0.7", "--top-k", "20"]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    outs = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert [o["prompt_token_ids"] for o in outs] == [list(b"hello"), list(b"page")]
    assert all(len(o["output_token_ids"]) == 5 and isinstance(o["text"], str) for o in outs)
