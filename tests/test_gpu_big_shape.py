"""The kernels that only real layer sizes reach (tensor-core attention with head size 64 and
four query heads per kv head, the decode GEMM with slices of K, the tcgen05 GEMM with its
fused gate, the 128k-wide output head), checked through the engine at the width of
Llama-3.2-1B with two layers and random weights, against the plain implementation."""

from __future__ import annotations

import pytest
import torch

import traces
from helpers import random_tokens, rel_err
from kvforge_b200 import PRESETS, ModelConfig
from kvforge_b200.models.folder import write_random_model
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    base = PRESETS["llama-3.2-1b"]
    cfg = ModelConfig(**{**base.__dict__, "num_layers": 2, "max_position_embeddings": 4096})
    folder = tmp_path_factory.mktemp("big") / "llama-1b-width-2-layers"
    # weights large enough that attention is not uniform: q.k has a spread of a few units
    write_random_model(folder, cfg, seed=5, store_dtype=torch.bfloat16, init_std=0.03, norm_std=0.05, device="cuda")
    reqs = {"a": random_tokens(cfg.vocab_size, 300, seed=1), "b": random_tokens(cfg.vocab_size, 97, seed=2)}
    plain = PlainLlama(folder, device="cuda")  # the plain implementation in 32-bit, run on the GPU for speed
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = {rid: plain.logits(t).cpu() for rid, t in reqs.items()}
    del plain
    torch.cuda.empty_cache()
    return folder, reqs, ref


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 6e-2)])
def test_llama_1b_width_whole_portions_and_decode(big, dtype, tol):
    from test_gpu_replay import check, replay_in_process

    folder, reqs, ref = big
    for steps in (traces.whole(reqs), traces.tail_one_by_one(reqs, 20), traces.mixed(reqs, {"a": 280, "b": 80}, max_live=2, seed=4)):
        outputs = replay_in_process(folder, dtype, steps)
        worst = check(steps, outputs, ref, tol)
        assert worst < tol


def test_llama_1b_width_bfloat16_is_no_worse_than_plain_bfloat16(big):
    from test_gpu_replay import MEAN_SLACK, check, replay_in_process

    folder, reqs, ref = big
    plain16 = PlainLlama(folder, dtype=torch.bfloat16, device="cuda")
    errs = []
    for rid, t in reqs.items():
        p16 = plain16.logits(t).cpu()
        errs += [rel_err(p16[i], ref[rid][i]) for i in range(len(t))]
    bound = MEAN_SLACK * sum(errs) / len(errs) + 5e-4
    steps = traces.whole(reqs)
    check(steps, replay_in_process(folder, "bfloat16", steps), ref, 6e-2, bound)


def test_llama_1b_width_generation_uses_graphs_and_the_device_token_loop(big):
    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    folder, reqs, ref = big
    prompts = [reqs["a"][:150], reqs["b"][:40], reqs["a"][150:170]]
    outs = {}
    for mode in ("graphs+async", "plain"):
        cfg = EngineConfig(
            cache=CacheConfig(block_size=16, num_blocks=64),
            scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=256, max_model_len=512),
            dtype="bfloat16", cuda_graphs=mode != "plain", async_output=mode != "plain",
        )  # fmt: skip
        engine = InferenceEngine(cfg, model=folder)
        res = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
        outs[mode] = [o.output_token_ids for o in res]
        assert all(len(o) == 12 for o in outs[mode])
    assert outs["graphs+async"] == outs["plain"]


def test_steps_of_many_tokens_replay_as_graphs_with_the_same_logits(big):
    """A step of more than 16 tokens is replayed as a CUDA graph made for its token count rounded up
    to 64 and its sequence count rounded up to a bucket (here at its first coming); the padding
    must change nothing."""
    from kvforge_b200 import CacheConfig
    from kvforge_b200.engine.core import EngineCore
    from kvforge_b200.engine.step import BatchItem

    folder, reqs, ref = big
    long, short = (reqs["a"] * 5)[:1300], reqs["b"]
    rows = {}
    for graphs in (False, True):
        core = EngineCore.from_model_dir(
            folder, dtype="bfloat16", cache=CacheConfig(block_size=16, num_blocks=100, watermark=0.0),
            max_num_seqs=4, max_num_batched_tokens=1024, max_model_len=1536, cuda_graphs=graphs,
        )  # fmt: skip
        core.runner.graph_after = 1
        bm = core.block_manager
        for rid, n in (("l", 650), ("s", len(short))):
            bm.allocate(rid, n)
            core.state_slots.allocate(rid)
        # 650 tokens of a long prompt beside a whole short one; then the rest of the long one beside a decoded token
        first = core.runner.step([BatchItem("l", long[:650], 0, "last"), BatchItem("s", short, 0, "last")]).float().cpu().clone()
        bm.append_slots("l", 1300, 650)
        bm.append_slots("s", len(short) + 1, len(short))
        second = core.runner.step([BatchItem("l", long[650:], 650, "last"), BatchItem("s", [7], len(short), "last")]).float().cpu().clone()
        rows[graphs] = (first, second)
        if graphs:
            assert core.runner.num_graph_kernels > 0 and len(core.runner.graph_kernels) >= 1
        core.rt.check_error_flag()
        del core
        torch.cuda.empty_cache()
    for a, b in zip(rows[False], rows[True]):
        for i in range(a.shape[0]):
            assert rel_err(b[i], a[i]) < 2e-2
    # and the short prompt's last row is what the plain implementation says
    assert rel_err(rows[True][0][1], ref["b"][len(short) - 1]) < 6e-2


@pytest.mark.parametrize("preset", ["llama-3.2-3b", "llama-3.1-8b"])
def test_wider_llamas_with_head_size_128(tmp_path_factory, preset):
    """The widths of Llama-3.2-3B (24 heads of 128 over 8 kv heads, hidden 3072) and Llama-3.1-8B
    (hidden 4096, intermediate 14336, untied head), two layers each: whole prompts, portions of
    changing size, portions beside decoded tokens, and the last tokens one by one, in 32-bit and in
    bfloat16 against the plain implementation."""
    from test_gpu_replay import check, replay_in_process

    base = PRESETS[preset]
    cfg = ModelConfig(**{**base.__dict__, "num_layers": 2, "max_position_embeddings": 4096})
    folder = tmp_path_factory.mktemp("wide") / f"{preset}-width-2-layers"
    write_random_model(folder, cfg, seed=6, store_dtype=torch.bfloat16, init_std=0.025, norm_std=0.05, device="cuda")
    reqs = {"a": random_tokens(cfg.vocab_size, 210, seed=3), "b": random_tokens(cfg.vocab_size, 66, seed=4)}
    plain = PlainLlama(folder, device="cuda")
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = {rid: plain.logits(t).cpu() for rid, t in reqs.items()}
    del plain
    torch.cuda.empty_cache()
    for dtype, tol in (("float32", 5e-5), ("bfloat16", 6e-2)):
        for steps in (traces.whole(reqs), traces.portions(reqs), traces.tail_one_by_one(reqs, 12), traces.mixed(reqs, {"a": 190, "b": 50}, max_live=2, seed=2)):
            outputs = replay_in_process(folder, dtype, steps)
            check(steps, outputs, ref, tol)


def test_llama_1b_whole_model_of_16_layers(tmp_path_factory):
    """Every layer of the Llama-3.2-1B shape (16 layers, tied head, llama3 scaling with factor 32),
    random weights: a few hundred tokens whole, in portions of changing size, with the last tokens
    one by one and two requests mixed, in 32-bit and bfloat16, against the plain implementation."""
    from test_gpu_replay import check, replay_in_process

    cfg = PRESETS["llama-3.2-1b"]
    assert cfg.num_layers == 16
    folder = tmp_path_factory.mktemp("whole") / "llama-1b-16-layers"
    write_random_model(folder, cfg, seed=8, store_dtype=torch.bfloat16, init_std=0.03, norm_std=0.05, device="cuda")
    reqs = {"a": random_tokens(cfg.vocab_size, 260, seed=5), "b": random_tokens(cfg.vocab_size, 75, seed=6)}
    plain = PlainLlama(folder, device="cuda")
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = {rid: plain.logits(t).cpu() for rid, t in reqs.items()}
    del plain
    torch.cuda.empty_cache()
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 8e-2)):
        for steps in (traces.whole(reqs), traces.portions(reqs), traces.tail_one_by_one(reqs, 16), traces.mixed(reqs, {"a": 240, "b": 60}, max_live=2, seed=3)):
            outputs = replay_in_process(folder, dtype, steps)
            check(steps, outputs, ref, tol)


@pytest.mark.parametrize("mode", ["float32", "bfloat16", "bfloat16-graphs"])
@pytest.mark.parametrize("live", [24, 64])
def test_llama_1b_width_many_requests_decoding_at_once(big, mode, live):
    """24 and 64 requests decoding at once at the width of Llama-3.2-1B (the batch-64 point of the
    benchmark): the library products of 17 to 64 rows, their slices of K, the graphs of the buckets
    32 and 64, key ranges of 512 once there are 256 pairs of sequence and kv head; requests leave
    and join on the way.  Logits stay on the device and are compared there."""
    import random

    from test_gpu_replay import run_trace

    folder, _, _ = big
    vocab = PRESETS["llama-3.2-1b"].vocab_size
    rng = random.Random(live)
    reqs = {f"m{i}": random_tokens(vocab, rng.randint(14, 36), seed=300 + i) for i in range(live + live // 2)}
    prompt_lens = {rid: max(1, len(t) - rng.randint(6, 10)) for rid, t in reqs.items()}
    plain = PlainLlama(folder, device="cuda")
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = {rid: plain.logits(t) for rid, t in reqs.items()}
    del plain
    steps = traces.many_decoders(reqs, prompt_lens, live, seed=live)
    dtype = mode.split("-")[0]
    tol = 5e-5 if dtype == "float32" else 6e-2
    outputs, runner = run_trace(folder, dtype, steps, max_live=64, to_host=False, cuda_graphs=mode.endswith("graphs"))
    rows = 0
    for s, places, got in zip(steps, traces.wanted_places(steps), outputs):
        assert got is not None and got.shape[0] == len(places)
        for i, (rid, pos) in enumerate(places):
            err = rel_err(got[i], ref[rid][pos])
            assert err < tol, f"step {s['step']} request {rid} position {pos}: error {err:.3e}"
            rows += 1
    assert rows > 10 * live
    if mode.endswith("graphs"):
        assert (64 if live > 32 else 32) in {key[1] for key in runner.core.runner._graphs if key[4]}
    del runner, outputs, ref
    torch.cuda.empty_cache()
