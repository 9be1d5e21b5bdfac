"""Each part alone against the plain function it stands for; a model whose execution list
names a layer twice and lets a layer read another's cache; attention with a window; and toy
parts defined here (a mixer with state of its own, a feed-forward that routes tokens to
experts, a position encoding with its own frequency table), registered, built and stepped
without any change to the framework's files."""

from __future__ import annotations

import json
import math

import pytest
import torch

import traces
from helpers import TINY, make_model_dir, random_tokens, rel_err
from plain_llama import PlainLlama, causal_attention, apply_rope, linear, plain_inv_freq, rms_norm, rope_cos_sin, swiglu

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 1e-5 if dtype == torch.float32 else 2.5e-2


def runtime(dtype, max_tokens=256):
    from kvforge_b200.engine.runtime import Runtime

    return Runtime("cuda", dtype, max_tokens, 8, 512)


def context(rt, seq_lens, starts, block_size, tables, slots):
    """A StepContext for hand-made batches: sequence i brings seq_lens[i] tokens from starts[i]."""
    from kvforge_b200.engine.runtime import StepContext
    import numpy as np

    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    positions = [p for n, s in zip(seq_lens, starts) for p in range(s, s + n)]
    qsl = [0]
    for n in seq_lens:
        qsl.append(qsl[-1] + n)
    ctx_lens = [s + n for n, s in zip(seq_lens, starts)]
    return StepContext(
        rt=rt, num_tokens=sum(seq_lens), num_seqs=len(seq_lens), token_ids=i32([0] * sum(seq_lens)), positions=i32(positions),
        query_start_loc=i32(qsl), context_lens=i32(ctx_lens), state_slots=i32(list(range(len(seq_lens)))), logit_rows=i32([0]),
        num_logit_rows=0, block_tables=[i32(tables)], slot_mappings=[i32(slots)], max_query_len=max(seq_lens),
        max_context_len=max(ctx_lens), block_size=block_size, h_query_start_loc=np.array(qsl), h_context_lens=np.array(ctx_lens),
        h_state_slots=np.arange(len(seq_lens)),
    )  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(dtype)
    part = build_part("norm", PartSpec("rmsnorm", {"dim": 100, "eps": 3e-6}), "x.")
    w = torch.rand(100) + 0.5
    part.bind({"weight": w.cuda()}, rt)
    resid, delta = torch.randn(9, 100), torch.randn(9, 100).to(dtype)
    r = resid.cuda()
    out = part.forward(None, r, delta.cuda())
    assert torch.allclose(out.float().cpu(), rms_norm(resid + delta.float(), w, 3e-6), atol=tol(dtype), rtol=tol(dtype))
    assert torch.allclose(r.cpu(), resid + delta.float(), atol=1e-6)


def test_rotary_part_table():
    from kvforge_b200.parts.base import PartSpec, build_part
    from plain_llama import llama3_scaled_inv_freq

    rt = runtime(torch.float32)
    scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    part = build_part("position", PartSpec("rotary", {"head_dim": 32, "theta": 500000.0, "scaling": scaling}))
    part.bind({}, rt)
    want = llama3_scaled_inv_freq(plain_inv_freq(32, 500000.0), 8.0, 1.0, 4.0, 64)
    assert torch.allclose(part.table().cpu(), want, rtol=1e-6)
    assert not torch.allclose(part.table().cpu(), plain_inv_freq(32, 500000.0), rtol=1e-3)
    plain_part = build_part("position", PartSpec("rotary", {"head_dim": 16, "theta": 10000.0}))
    plain_part.bind({}, rt)
    assert torch.equal(plain_part.table().cpu(), plain_inv_freq(16, 10000.0))


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(dtype)
    h, i = 80, 112
    part = build_part("ffn", PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": i, "activation": "silu"}), "m.")
    wg, wu, wd = (torch.randn(i, h) * 0.2).to(dtype), (torch.randn(i, h) * 0.2).to(dtype), (torch.randn(h, i) * 0.2).to(dtype)
    part.bind({"gate_proj.weight": wg.cuda(), "up_proj.weight": wu.cuda(), "down_proj.weight": wd.cuda()}, rt)
    x = torch.randn(13, h).to(dtype)
    out = part.forward(None, x.cuda())
    ref = swiglu(x.float(), wg.float(), wu.float(), wd.float())
    assert rel_err(out.float().cpu(), ref) < tol(dtype)
    with pytest.raises(ValueError):
        build_part("ffn", PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": i, "activation": "gelu"}))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 7])
def test_paged_attention_part(dtype, window):
    """Whole prompt in one step, then a portion and single tokens on top of the cache."""
    from kvforge_b200.parts.base import LayerCache, PartSpec, build_part

    rt = runtime(dtype)
    h, nh, nkv, d, bs = 80, 6, 3, 48, 4
    pos = PartSpec("rotary", {"head_dim": d, "theta": 25000.0})
    part = build_part("mixer", PartSpec("paged_attention", {"hidden_size": h, "num_heads": nh, "num_kv_heads": nkv, "head_dim": d, "position": pos, "window": window}), "a.")
    w = {n: (torch.randn(o, i) * 0.15).to(dtype) for n, (o, i) in {"q_proj.weight": (nh * d, h), "k_proj.weight": (nkv * d, h), "v_proj.weight": (nkv * d, h), "o_proj.weight": (h, nh * d)}.items()}
    part.bind({k: v.cuda() for k, v in w.items()}, rt)
    t = 30
    x = torch.randn(t, h).to(dtype)
    # plain: the formulas of the attention layer on the whole sequence
    cos, sin = rope_cos_sin(torch.arange(t), plain_inv_freq(d, 25000.0))
    xf = x.float()
    q = apply_rope(linear(xf, w["q_proj.weight"].float()).view(t, nh, d), cos, sin)
    k = apply_rope(linear(xf, w["k_proj.weight"].float()).view(t, nkv, d), cos, sin)
    v = linear(xf, w["v_proj.weight"].float()).view(t, nkv, d)
    ref = linear(causal_attention(q, k, v, 1 / math.sqrt(d), window).reshape(t, -1), w["o_proj.weight"].float())
    nb = 12
    table = [7, 2, 9, 0, 11, 4, 5, 1]
    slots = [table[p // bs] * bs + p % bs for p in range(t)]
    cache = LayerCache(torch.zeros(nb, nkv, bs, d, device="cuda", dtype=dtype), torch.zeros(nb, nkv, bs, d, device="cuda", dtype=dtype), 0)
    cuts = [(0, 17), (17, 26), (26, 27), (27, 28), (28, 30)]
    got = []
    for a, b in cuts:
        ctx = context(rt, [b - a], [a], bs, [table], slots[a:b])
        got.append(part.forward(ctx, x[a:b].cuda(), cache).float().cpu().clone())
    assert rel_err(torch.cat(got), ref) < tol(dtype)
    assert part.cache_need().kind == ("window" if window else "full")


def _variant_folder(tmp_path, name, extra):
    d = make_model_dir(tmp_path, name, store_dtype=torch.bfloat16)
    cfg = json.loads((d / "config.json").read_text())
    cfg.update(extra)
    (d / "config.json").write_text(json.dumps(cfg))
    return d


@pytest.fixture
def variant_architecture():
    """A test-only architecture: the Llama parts, with the order of layers and an attention
    window taken from extra config.json keys."""
    from kvforge_b200 import ModelConfig
    from kvforge_b200.config.registry import register_architecture, unregister_architecture
    from kvforge_b200.models.llama import llama_spec
    from kvforge_b200.parts.model import LayerCall

    def parse(d):
        cfg = ModelConfig.from_hf_dict(d)
        cfg.extra = {"execution": d.get("test_execution"), "window": d.get("test_window")}
        return cfg

    def build(cfg):
        spec = llama_spec(cfg)
        if cfg.extra["execution"]:
            spec.execution = [LayerCall(layer, src) for layer, src in cfg.extra["execution"]]
            spec.__post_init__()
        if cfg.extra["window"]:
            for ls in spec.layers[1:]:  # layer 0 keeps every key, the others a window: two cache groups
                mixer = ls.block.params["mixer"]
                ls.block.params["mixer"] = type(mixer)(mixer.kind, {**mixer.params, "window": cfg.extra["window"]})
        return spec

    register_architecture("TestVariantForCausalLM", parse, build)
    yield "TestVariantForCausalLM"
    unregister_architecture("TestVariantForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_execution_list_names_a_layer_twice_and_shares_a_cache(tmp_path, variant_architecture, dtype):
    from test_gpu_replay import MEAN_SLACK, TOL, check, plain_bfloat16_mean_error, replay_in_process

    execution = [[0, None], [1, None], [0, None], [2, 1], [1, 2]]
    folder = _variant_folder(tmp_path, "tiny-b", {"architectures": [variant_architecture], "test_execution": execution})
    plain = PlainLlama(folder)
    plain.execution = [(layer, src) for layer, src in execution]
    reqs = {f"r{i}": random_tokens(320, n, seed=i) for i, n in enumerate([45, 9, 70])}
    ref = {rid: plain.logits(t) for rid, t in reqs.items()}
    assert rel_err(ref["r0"], PlainLlama(folder).logits(reqs["r0"])) > 1e-2  # the order matters
    mean_tol = None
    if dtype == "bfloat16":
        plain16 = PlainLlama(folder, dtype=torch.bfloat16)
        plain16.execution = plain.execution
        mean_tol = MEAN_SLACK * plain_bfloat16_mean_error(plain16, reqs, ref) + 5e-4
    for steps in (traces.whole(reqs), traces.portions(reqs), traces.mixed(reqs, {r: len(t) - 10 for r, t in reqs.items()}, seed=1)):
        check(steps, replay_in_process(folder, dtype, steps), ref, TOL[dtype], mean_tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_have_pages_of_their_own(tmp_path, variant_architecture, dtype):
    from kvforge_b200.replay import TraceRunner
    from test_gpu_replay import TOL, check

    folder = _variant_folder(tmp_path, "tiny-c", {"architectures": [variant_architecture], "test_window": 21})
    reqs = {f"r{i}": random_tokens(203, n, seed=i) for i, n in enumerate([150, 40, 97])}

    class WindowedPlain(PlainLlama):
        def attention(self, layer, x, positions, kv=None):
            self.window = None if layer == 0 else 21
            return super().attention(layer, x, positions, kv)

    plain = WindowedPlain(folder)
    ref = {rid: plain.logits(t) for rid, t in reqs.items()}
    assert rel_err(ref["r0"], PlainLlama(folder).logits(reqs["r0"])) > 1e-3
    cuts = {"whole": traces.whole(reqs), "portions": traces.portions(reqs), "tail": traces.tail_one_by_one(reqs, 32),
            "mixed": traces.mixed(reqs, {r: len(t) - 12 for r, t in reqs.items()}, seed=3)}  # fmt: skip
    for cut, steps in cuts.items():
        runner = TraceRunner(str(folder), dtype, traces.tokens_needed(steps))
        bm = runner.core.block_manager
        assert bm.num_groups == 2
        window_group = [g for g in range(2) if bm.group_specs[g].kind == "window"][0]
        outs, most_saved = [], 0
        for s in steps:
            o = runner.step(s)
            outs.append(None if o is None else o.clone())
            bm.check_invariants()
            most_saved = max(most_saved, bm.free_blocks_of(window_group) - bm.free_blocks_of(1 - window_group))
        check(steps, outs, ref, TOL[dtype])
        if cut != "whole":  # pages behind the window were given back while the full group kept its own
            assert most_saved >= 5, cut  # 150 tokens are 10 pages of 16; a window of 21 needs 3


@pytest.mark.parametrize("name,window", [("tiny-d", 40), ("tiny-e", 70)])
@pytest.mark.parametrize("graphs", [False, True])
def test_a_window_through_the_tensor_core_kernels(tmp_path, variant_architecture, name, window, graphs):
    """The same arrangement (layer 0 sees every key, the others a window) with head sizes 64 and
    128 in bfloat16, where prompts and portions run on the tcgen05 kernel and single tokens on the
    TMA kernel, at the model's own page size, eager and as captured graphs: a window that ends
    inside a key tile, inside a page, and behind pages that were given back."""
    from test_gpu_replay import TOL, check, run_trace

    folder = _variant_folder(tmp_path, name, {"architectures": [variant_architecture], "test_window": window})
    vocab = TINY[name]["cfg"].vocab_size
    reqs = {f"r{i}": random_tokens(vocab, n, seed=40 + i) for i, n in enumerate([190, 33, 121])}

    class WindowedPlain(PlainLlama):
        def attention(self, layer, x, positions, kv=None):
            self.window = None if layer == 0 else window
            return super().attention(layer, x, positions, kv)

    plain = WindowedPlain(folder)
    ref = {rid: plain.logits(t) for rid, t in reqs.items()}
    assert rel_err(ref["r0"], PlainLlama(folder).logits(reqs["r0"])) > 1e-3
    cuts = (traces.whole(reqs), traces.portions(reqs), traces.tail_one_by_one(reqs, 32), traces.mixed(reqs, {r: len(t) - 12 for r, t in reqs.items()}, seed=3))
    for steps in cuts:
        steps = traces.last_only(steps) if graphs else steps
        outs, runner = run_trace(folder, "bfloat16", steps, block_size=TINY[name]["block_size"], cuda_graphs=graphs)
        check(steps, outs, ref, TOL["bfloat16"])
        runner.core.rt.check_error_flag()


DECAY = 0.9
TOY_STATE = 24


def toy_state_architecture():
    """Registers (once) a mixer that keeps a decaying sum per request (no keys, no pages), written
    here with torch operations, and returns the builder of a model whose odd layers use it while
    its even layers keep attention: state slots and pages in one model.  Everything goes through
    the public registries; no file of the framework knows of it.

    The mixer works on the device alone, with shapes that depend only on the step's capacity, so
    that a step can be captured as a CUDA graph: which sequence a token belongs to comes from
    ``query_start_loc``; a token outside every sequence (padding of a captured shape) and a
    sequence without queries or without a slot (``state_slots[b] < 0``) touch no state."""
    from kvforge_b200.models.llama import llama_spec
    from kvforge_b200.parts.base import MIXERS, CacheNeed, Mixer, PartSpec, WeightDecl, register_mixer

    class DecayingSum(Mixer):
        """state_t = DECAY * state_{t-1} + x_t W_in^T ;  y_t = state_t W_out^T"""

        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.h, self.s = params["hidden_size"], params["state_size"]

        @classmethod
        def weight_decls(cls, params):
            return {"in_proj.weight": WeightDecl((params["state_size"], params["hidden_size"])),
                    "out_proj.weight": WeightDecl((params["hidden_size"], params["state_size"]))}  # fmt: skip

        def cache_need(self):
            return CacheNeed("none")

        def state_shape(self):
            return (self.s,)

        def bind(self, weights, rt):
            super().bind(weights, rt)
            self.w_in, self.w_out = weights["in_proj.weight"].float(), weights["out_proj.weight"].float()

        def forward(self, ctx, x, cache):
            n, nb = x.shape[0], ctx.num_seqs
            u = x.float() @ self.w_in.t()
            qsl = ctx.query_start_loc.long()
            tok = torch.arange(n, device=x.device)
            seq = torch.searchsorted(qsl[1:].contiguous(), tok, right=True).clamp(max=nb - 1)  # how many sequences end at or before the token
            slot = ctx.state_slots.long()[seq]
            live = (tok < qsl[nb]) & (slot >= 0)
            slot = slot.clamp(min=0)
            # y_t = DECAY^(t - first + 1) * state + sum over the sequence's tokens s <= t of DECAY^(t - s) * u_s
            lag = tok[:, None] - tok[None, :]
            same = (seq[:, None] == seq[None, :]) & (lag >= 0) & live[:, None] & live[None, :]
            mix = torch.where(same, DECAY ** lag.clamp(min=0).float(), torch.zeros((), device=x.device))
            before = cache.state[slot]
            y = mix @ u + (DECAY ** (tok - qsl[seq] + 1).clamp(min=0).float())[:, None] * before
            y = torch.where(live[:, None], y, torch.zeros((), device=x.device))
            # the state after the step is y at a sequence's last token; slots of other requests stay as they are
            last = live & (tok == qsl[seq + 1] - 1)
            pick = (last[None, :] & (slot[None, :] == torch.arange(cache.state.shape[0], device=x.device)[:, None])).float()
            cache.state.copy_(torch.where(pick.sum(1, keepdim=True) > 0, pick @ y, cache.state))
            return (y @ self.w_out.t()).to(x.dtype)

    if "decaying_sum" not in MIXERS:
        register_mixer("decaying_sum")(DecayingSum)

    def build(cfg):
        spec = llama_spec(cfg)
        for i, ls in enumerate(spec.layers):
            if i % 2 == 1:  # odd layers keep a state, even layers keep keys: both kinds in one model
                ls.block.params["mixer"] = PartSpec("decaying_sum", {"hidden_size": cfg.hidden_size, "state_size": TOY_STATE})
                ls.block.params["mixer_name"] = "toy"
        return spec

    return build


class ToyStatePlain(PlainLlama):
    """The plain model with the decaying sum in its odd layers, token by token."""

    def attention(self, layer, x, positions, kv=None):
        if layer % 2 == 0:
            return super().attention(layer, x, positions, kv)
        u = x.float() @ self.w[f"layers.{layer}.toy.in_proj.weight"].float().t()
        state = torch.zeros(TOY_STATE)
        rows = []
        for t in range(x.shape[0]):
            state = DECAY * state + u[t]
            rows.append(state)
        return (torch.stack(rows) @ self.w[f"layers.{layer}.toy.out_proj.weight"].float().t()).to(x.dtype), None


def toy_state_folder(tmp_path, build, store_dtype):
    from kvforge_b200.parts.model import DecoderModel
    from kvforge_b200.weights.random_init import write_model_dir

    cfg = TINY["tiny-b"]["cfg"]
    cj = cfg.to_hf_dict()
    cj["architectures"] = ["ToyStateForCausalLM"]
    model = DecoderModel(build(cfg))
    assert model.state_shapes == [None, (TOY_STATE,), None] and len(model.groups) == 1 and len(model.groups[0].calls) == 2
    return write_model_dir(tmp_path / "toy", cj, model.expected_weights(), seed=5, store_dtype=store_dtype, init_std=0.1, norm_std=0.1)


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from kvforge_b200 import ModelConfig
    from kvforge_b200.config.registry import register_architecture, unregister_architecture
    from kvforge_b200.replay import TraceRunner
    from test_gpu_replay import check

    build = toy_state_architecture()
    register_architecture("ToyStateForCausalLM", ModelConfig.from_hf_dict, build)
    try:
        folder = toy_state_folder(tmp_path, build, torch.float32)
        plain = ToyStatePlain(folder)
        reqs = {f"r{i}": random_tokens(320, n, seed=i) for i, n in enumerate([33, 5, 48, 20, 27])}
        ref = {rid: plain.logits(t) for rid, t in reqs.items()}
        cuts = (traces.whole(reqs), traces.portions(reqs), traces.tail_one_by_one(reqs, 12), traces.mixed(reqs, {r: len(t) - 6 for r, t in reqs.items()}, max_live=3, seed=2))
        for graphs in (False, True):
            for steps in cuts:
                if graphs:
                    steps = traces.last_only(steps)
                runner = TraceRunner(str(folder), "float32", traces.tokens_needed(steps), max_live=3, block_size=8, cuda_graphs=graphs)
                outs = []
                for s in steps:
                    o = runner.step(s)
                    outs.append(None if o is None else o.clone())
                check(steps, outs, ref, 2e-5)  # slots are used again: a new request must start from zero
                runner.core.state_slots.check_invariants()
                if graphs and steps is not cuts[0]:
                    assert runner.core.runner.num_graph_kernels > 0
    finally:
        unregister_architecture("ToyStateForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_toy_mixers_state_survives_graphs_chunked_prefill_and_preemption_in_the_engine(tmp_path, dtype):
    """The same toy model through ``InferenceEngine`` with CUDA graphs: prompts cut into portions
    by a small token budget, four state slots for six requests, and so few pages that running
    requests are preempted and recomputed (their slot is given back and a fresh one starts from
    zero).  A step on which a graph is captured must advance the state once, not twice.  Tokens
    are the plain model's: all of them in 32-bit, in bfloat16 wherever its top-2 margin is
    larger than bfloat16 rounding."""
    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, ModelConfig, SamplingParams, SchedulerConfig
    from kvforge_b200.config.registry import register_architecture, unregister_architecture

    build = toy_state_architecture()
    register_architecture("ToyStateForCausalLM", ModelConfig.from_hf_dict, build)
    try:
        folder = toy_state_folder(tmp_path, build, torch.bfloat16)
        plain = ToyStatePlain(folder)
        prompts = [random_tokens(320, n, seed=60 + i) for i, n in enumerate([33, 21, 40, 18, 27, 36])]
        cfg = EngineConfig(
            cache=CacheConfig(block_size=8, num_blocks=18),
            scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=24, max_model_len=128),
            dtype=dtype, cuda_graphs=True,
        )  # fmt: skip
        engine = InferenceEngine(cfg, model=folder)
        outs = engine.generate(prompts, SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True))
        assert engine.scheduler.num_preemptions > 0
        assert engine.runner.num_graph_kernels > 0 and any(key[4] for key in engine.runner._graphs) and any(not key[4] for key in engine.runner._graphs)
        engine.core.rt.check_error_flag()
        engine.core.state_slots.check_invariants()
        assert engine.block_manager.num_free_blocks == 18
        checked = 0
        for p, o in zip(prompts, outs):
            assert o.finished and len(o.output_token_ids) == 20
            if dtype == "float32":
                assert o.output_token_ids == plain.greedy(p, 20)
                checked += 20
                continue
            ids = list(p)
            for tok in o.output_token_ids:
                logits = plain.logits(ids)[-1]
                top = logits.topk(2).values
                if float(top[0] - top[1]) > 0.08 * float(logits.abs().max()):
                    assert tok == int(logits.argmax())
                    checked += 1
                ids.append(tok)  # the plain model follows the engine's tokens, so a close call costs one comparison
        assert checked > 40
    finally:
        unregister_architecture("ToyStateForCausalLM")


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_are_registered_built_and_stepped(tmp_path):
    """A feed-forward that routes each token to two of four experts, and a position encoding
    with a frequency table of its own, both written here and plugged in through the public
    registries only; odd layers route, even layers keep the dense feed-forward."""
    from kvforge_b200 import ModelConfig
    from kvforge_b200.config.registry import register_architecture, unregister_architecture
    from kvforge_b200.models.llama import llama_spec
    from kvforge_b200.parts.base import (
        FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PartSpec, PositionEncoding, WeightDecl, register_feed_forward, register_position_encoding,
    )  # fmt: skip
    from kvforge_b200.replay import TraceRunner
    from test_gpu_replay import check

    n_experts, top, inter = 4, 2, 40

    def routed(x, router, up, down):
        """softmax over the chosen experts' router logits (32-bit), experts are x -> relu(x U^T) D^T"""
        logits = x.float() @ router.float().t()
        val, idx = logits.topk(top, dim=-1)
        gate = torch.softmax(val, dim=-1)
        out = torch.zeros_like(x, dtype=torch.float32)
        for e in range(n_experts):
            y = torch.relu(x.float() @ up[e].float().t()) @ down[e].float().t()
            w = (gate * (idx == e)).sum(-1, keepdim=True)
            out += w * y
        return out

    class Routed(FeedForward):
        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)

        @classmethod
        def weight_decls(cls, params):
            h = params["hidden_size"]
            return {
                "router.weight": WeightDecl((n_experts, h)),
                "experts.up": WeightDecl((n_experts, inter, h)),
                "experts.down": WeightDecl((n_experts, h, inter)),
            }

        def bind(self, weights, rt):
            super().bind(weights, rt)
            self.router, self.up, self.down = weights["router.weight"], weights["experts.up"], weights["experts.down"]

        def forward(self, ctx, x):
            return routed(x, self.router, self.up, self.down).to(x.dtype)

    class LinearFrequencies(PositionEncoding):
        """pair j turns by pos * base / (j + 1)"""

        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.table_host = float(params["base"]) / torch.arange(1, int(params["head_dim"]) // 2 + 1, dtype=torch.float32)

        def bind(self, weights, rt):
            super().bind(weights, rt)
            self.dev = self.table_host.to(rt.device).contiguous()

        def table(self):
            return self.dev

    if "toy_routed" not in FEED_FORWARDS:
        register_feed_forward("toy_routed")(Routed)
    if "toy_linear_frequencies" not in POSITION_ENCODINGS:
        register_position_encoding("toy_linear_frequencies")(LinearFrequencies)

    def build(cfg):
        spec = llama_spec(cfg)
        position = PartSpec("toy_linear_frequencies", {"head_dim": cfg.head_dim, "base": 0.7})
        for i, ls in enumerate(spec.layers):
            mixer = ls.block.params["mixer"]
            ls.block.params["mixer"] = PartSpec(mixer.kind, {**mixer.params, "position": position})
            if i % 2 == 1:
                ls.block.params["ffn"] = PartSpec("toy_routed", {"hidden_size": cfg.hidden_size})
                ls.block.params["ffn_name"] = "moe"
        return spec

    register_architecture("ToyRoutedForCausalLM", ModelConfig.from_hf_dict, build)
    try:
        from kvforge_b200.parts.model import DecoderModel
        from kvforge_b200.weights.random_init import write_model_dir

        cfg = TINY["tiny-b"]["cfg"]
        cj = cfg.to_hf_dict()
        cj["architectures"] = ["ToyRoutedForCausalLM"]
        model = DecoderModel(build(cfg))
        folder = write_model_dir(tmp_path / "toy", cj, model.expected_weights(), seed=6, store_dtype=torch.float32, init_std=0.1, norm_std=0.1)

        class ToyPlain(PlainLlama):
            def __init__(self, *a, **k):
                super().__init__(*a, **k)
                self.inv_freq = 0.7 / torch.arange(1, self.d // 2 + 1, dtype=torch.float32)

            def mlp(self, layer, x):
                if layer % 2 == 0:
                    return super().mlp(layer, x)
                p = f"layers.{layer}.moe."
                return routed(x, self.w[p + "router.weight"], self.w[p + "experts.up"], self.w[p + "experts.down"])

        plain = ToyPlain(folder)
        reqs = {f"r{i}": random_tokens(320, n, seed=10 + i) for i, n in enumerate([33, 5, 48, 20, 27])}
        ref = {rid: plain.logits(t) for rid, t in reqs.items()}
        for steps in (traces.whole(reqs), traces.portions(reqs), traces.tail_one_by_one(reqs, 12), traces.mixed(reqs, {r: len(t) - 6 for r, t in reqs.items()}, max_live=3, seed=2)):
            runner = TraceRunner(str(folder), "float32", traces.tokens_needed(steps), max_live=3)
            outs = []
            for s in steps:
                o = runner.step(s)
                outs.append(None if o is None else o.clone())
            check(steps, outs, ref, 2e-5)
    finally:
        unregister_architecture("ToyRoutedForCausalLM")


def test_a_toy_position_encoding_added_at_the_embedding_and_attention_without_rotation(tmp_path):
    """Learned absolute positions: a table of its own tensor, added to the residual stream after
    the embedding lookup; the attention layers get no position encoding at all and leave queries
    and keys as projected.  Both through the public registries and ``ModelSpec`` alone, in 32-bit
    and bfloat16, eager and as captured graphs."""
    from kvforge_b200 import ModelConfig
    from kvforge_b200.config.registry import register_architecture, unregister_architecture
    from kvforge_b200.models.llama import llama_spec
    from kvforge_b200.parts.base import POSITION_ENCODINGS, PartSpec, PositionEncoding, WeightDecl, register_position_encoding
    from kvforge_b200.parts.model import DecoderModel
    from kvforge_b200.weights.random_init import write_model_dir
    from test_gpu_replay import TOL, check, run_trace

    max_pos = 160

    class LearnedPositions(PositionEncoding):
        @classmethod
        def weight_decls(cls, params):
            return {"weight": WeightDecl((int(params["max_positions"]), int(params["hidden_size"])))}

        def bind(self, weights, rt):
            super().bind(weights, rt)
            self.weight = weights["weight"].float()

        def embed(self, ctx, resid):
            resid.add_(self.weight[ctx.positions.long()])

    if "toy_learned_positions" not in POSITION_ENCODINGS:
        register_position_encoding("toy_learned_positions")(LearnedPositions)

    def build(cfg):
        spec = llama_spec(cfg)
        for ls in spec.layers:
            mixer = ls.block.params["mixer"]
            ls.block.params["mixer"] = PartSpec(mixer.kind, {**mixer.params, "position": None})
        spec.input_position = PartSpec("toy_learned_positions", {"max_positions": max_pos, "hidden_size": cfg.hidden_size})
        return spec

    register_architecture("ToyLearnedPositionsForCausalLM", ModelConfig.from_hf_dict, build)
    try:
        cfg = TINY["tiny-d"]["cfg"]
        cj = cfg.to_hf_dict()
        cj["architectures"] = ["ToyLearnedPositionsForCausalLM"]
        model = DecoderModel(build(cfg))
        assert "model.embed_positions.weight" in model.expected_weights()
        assert cfg.tie_word_embeddings  # so the folder holds no separate output head
        folder = write_model_dir(tmp_path / "toy", cj, model.expected_weights(), seed=9, store_dtype=torch.bfloat16, init_std=0.1, norm_std=0.1, skip=("lm_head.weight",))

        class ToyPlain(PlainLlama):
            def __init__(self, *a, **k):
                super().__init__(*a, **k)
                self.inv_freq = torch.zeros(self.d // 2)  # angle 0: no rotation

            def embed(self, ids):
                return super().embed(ids) + self.w["embed_positions.weight"][: ids.shape[0]]

        plain = ToyPlain(folder)
        reqs = {f"r{i}": random_tokens(cfg.vocab_size, n, seed=20 + i) for i, n in enumerate([70, 5, 130, 33])}
        ref = {rid: plain.logits(t) for rid, t in reqs.items()}
        # positions matter: the same tokens in another order give other logits at the last place
        swapped = list(reqs["r0"])
        swapped[3], swapped[40] = swapped[40], swapped[3]
        assert rel_err(plain.logits(swapped)[-1], ref["r0"][-1]) > 1e-3
        cuts = (traces.whole(reqs), traces.portions(reqs), traces.tail_one_by_one(reqs, 12), traces.mixed(reqs, {r: max(1, len(t) - 6) for r, t in reqs.items()}, max_live=3, seed=2))
        for dtype in ("float32", "bfloat16"):
            for graphs in (False, True):
                for steps in cuts:
                    steps = traces.last_only(steps) if graphs else steps
                    outs, _ = run_trace(folder, dtype, steps, max_live=3, cuda_graphs=graphs)
                    check(steps, outs, ref, TOL[dtype])
    finally:
        unregister_architecture("ToyLearnedPositionsForCausalLM")


def test_a_toy_embedding_and_a_toy_head_are_registered_built_and_stepped(tmp_path):
    """An embedding that scales its rows by the square root of the width and a head that caps its
    logits softly (``cap * tanh(logits / cap)``), both written here on top of the built-in parts and
    named in ``ModelSpec.embedding`` / ``ModelSpec.head``: what turns tokens into the residual
    stream and rows into logits is a part like any other."""
    from kvforge_b200 import ModelConfig
    from kvforge_b200.config.registry import register_architecture, unregister_architecture
    from kvforge_b200.models.llama import llama_spec
    from kvforge_b200.parts.base import EMBEDDINGS, HEADS, PartSpec, register_embedding, register_head
    from kvforge_b200.parts.embedding import TokenEmbedding
    from kvforge_b200.parts.head import LinearHead
    from kvforge_b200.parts.model import DecoderModel
    from kvforge_b200.weights.random_init import write_model_dir
    from test_gpu_replay import TOL, check, run_trace

    cap = 3.0

    class ScaledEmbedding(TokenEmbedding):
        def forward(self, ctx, resid):
            super().forward(ctx, resid)
            resid.mul_(math.sqrt(self.hidden))

    class SoftCappedHead(LinearHead):
        def forward(self, ctx, x):
            logits = super().forward(ctx, x)
            return logits.copy_(cap * torch.tanh(logits / cap))

    if "toy_scaled_embedding" not in EMBEDDINGS:
        register_embedding("toy_scaled_embedding")(ScaledEmbedding)
    if "toy_soft_capped_head" not in HEADS:
        register_head("toy_soft_capped_head")(SoftCappedHead)

    def build(cfg):
        spec = llama_spec(cfg)
        sizes = {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}
        spec.embedding = PartSpec("toy_scaled_embedding", sizes)
        spec.head = PartSpec("toy_soft_capped_head", sizes)
        return spec

    register_architecture("ToyEndsForCausalLM", ModelConfig.from_hf_dict, build)
    try:
        for name in ("tiny-a", "tiny-b"):  # a tied head and one with a tensor of its own
            cfg = TINY[name]["cfg"]
            cj = cfg.to_hf_dict()
            cj["architectures"] = ["ToyEndsForCausalLM"]
            model = DecoderModel(build(cfg))
            skip = ("lm_head.weight",) if cfg.tie_word_embeddings else ()
            folder = write_model_dir(tmp_path / name, cj, model.expected_weights(), seed=12, store_dtype=torch.bfloat16, init_std=0.05, norm_std=0.1, skip=skip)

            class ToyPlain(PlainLlama):
                def embed(self, ids):
                    return super().embed(ids) * math.sqrt(self.hidden)

                def logits(self, ids):
                    return cap * torch.tanh(super().logits(ids) / cap)

            plain = ToyPlain(folder)
            reqs = {f"r{i}": random_tokens(cfg.vocab_size, n, seed=30 + i) for i, n in enumerate([40, 5, 70])}
            ref = {rid: plain.logits(t) for rid, t in reqs.items()}
            assert float(ref["r0"].abs().max()) > 0.5 * cap  # the cap bites
            cuts = (traces.whole(reqs), traces.tail_one_by_one(reqs, 12), traces.mixed(reqs, {r: max(1, len(t) - 6) for r, t in reqs.items()}, max_live=3, seed=2))
            for dtype in ("float32", "bfloat16"):
                for graphs in (False, True):
                    for steps in cuts:
                        steps = traces.last_only(steps) if graphs else steps
                        outs, _ = run_trace(folder, dtype, steps, max_live=3, block_size=TINY[name]["block_size"], cuda_graphs=graphs)
                        check(steps, outs, ref, TOL[dtype])
    finally:
        unregister_architecture("ToyEndsForCausalLM")


def test_a_toy_norm_and_a_toy_block_arrangement_are_registered_built_and_stepped(tmp_path):
    """A norm that centres its rows and has a bias, and an arrangement in which the mixer and the
    feed-forward read the same normed rows and both add to the stream
    (``h = h + mixer(n(h)) + ffn(n(h))``, one norm a layer), both written here and plugged in
    through the public registries only; the final norm is the toy one too.  The arrangement asks
    its parts for their results as tensors (``ctx.residual = None`` around their calls) and takes
    whatever form they come in.  In 32-bit and bfloat16, eager and as captured graphs."""
    from kvforge_b200 import ModelConfig, ops
    from kvforge_b200.config.registry import register_architecture, unregister_architecture
    from kvforge_b200.models.llama import llama_spec
    from kvforge_b200.parts.base import BLOCKS, NORMS, Block, Norm, PartSpec, WeightDecl, build_part, register_block, register_norm
    from kvforge_b200.parts.model import DecoderModel
    from kvforge_b200.weights.random_init import write_model_dir
    from test_gpu_replay import TOL, check, run_trace

    def centred(v, w, b, eps):
        v = v.float()
        v = v - v.mean(-1, keepdim=True)
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float() + b.float()

    def as_float(y, n):
        """A part's result as float rows, whichever form it came in."""
        if isinstance(y, ops.Partials):
            return y.t[:, :n].sum(0)
        assert y is not ops.ADDED and y is not None
        return y[:n].float()

    class CentredNorm(Norm):
        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.dim, self.eps = int(params["dim"]), float(params["eps"])

        @classmethod
        def weight_decls(cls, params):
            d = int(params["dim"])
            return {"weight": WeightDecl((d,), kind="vector", init="ones"), "bias": WeightDecl((d,), kind="vector")}

        def bind(self, weights, rt):
            super().bind(weights, rt)
            self.weight, self.bias = weights["weight"], weights["bias"]

        def forward(self, ctx, resid, delta, rows=None, num_rows=None):
            if delta is not None and delta is not ops.ADDED:
                assert rows is None
                resid += as_float(delta, resid.shape[0])
            v = resid if rows is None else resid[rows[:num_rows].long()]
            return centred(v, self.weight, self.bias, self.eps).to(self.rt.dtype)

    class ParallelBlock(Block):
        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.norm = build_part("norm", params["norm"], f"{prefix}input_layernorm.")
            self.mixer = build_part("mixer", params["mixer"], f"{prefix}self_attn.")
            self.ffn = build_part("ffn", params["ffn"], f"{prefix}mlp.")

        def sub_parts(self):
            return [self.norm, self.mixer, self.ffn]

        def mixer_part(self):
            return self.mixer

        def forward(self, ctx, resid, delta, cache):
            n = resid.shape[0]
            x = self.norm.forward(ctx, resid, delta)
            stream, ctx.residual = ctx.residual, None  # both parts read x: neither may add into the stream yet
            a = as_float(self.mixer.forward(ctx, x, cache), n)
            f = as_float(self.ffn.forward(ctx, x), n)
            ctx.residual = stream
            resid += a + f
            return None

    if "toy_centred_norm" not in NORMS:
        register_norm("toy_centred_norm")(CentredNorm)
    if "toy_parallel" not in BLOCKS:
        register_block("toy_parallel")(ParallelBlock)

    def build(cfg):
        spec = llama_spec(cfg)
        norm = PartSpec("toy_centred_norm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps})
        for ls in spec.layers:
            ls.block = PartSpec("toy_parallel", {"norm": norm, "mixer": ls.block.params["mixer"], "ffn": ls.block.params["ffn"]})
        spec.final_norm = norm
        return spec

    register_architecture("ToyParallelForCausalLM", ModelConfig.from_hf_dict, build)
    try:
        cfg = TINY["tiny-d"]["cfg"]
        cj = cfg.to_hf_dict()
        cj["architectures"] = ["ToyParallelForCausalLM"]
        model = DecoderModel(build(cfg))
        names = model.expected_weights()
        assert "model.layers.0.input_layernorm.bias" in names and "model.norm.bias" in names
        assert not any("post_attention_layernorm" in k for k in names)
        folder = write_model_dir(tmp_path / "toy", cj, names, seed=12, store_dtype=torch.bfloat16, init_std=0.1, norm_std=0.1, skip=("lm_head.weight",))

        class ToyPlain(PlainLlama):
            def hidden_states(self, ids):
                ids = torch.as_tensor(ids, dtype=torch.long)
                positions = torch.arange(ids.shape[0])
                h = self.embed(ids).float()
                for layer, _ in self.execution:
                    p = f"layers.{layer}.input_layernorm."
                    x = centred(h, self.w[p + "weight"], self.w[p + "bias"], self.eps)
                    a, _ = self.attention(layer, x, positions, None)
                    h = h + a + self.mlp(layer, x)
                return centred(h, self.w["norm.weight"], self.w["norm.bias"], self.eps)

        plain = ToyPlain(folder)
        reqs = {f"r{i}": random_tokens(cfg.vocab_size, n, seed=40 + i) for i, n in enumerate([70, 5, 130, 33])}
        ref = {rid: plain.logits(t) for rid, t in reqs.items()}
        # the bias matters: without it the same model gives other logits
        saved = plain.w["norm.bias"].clone()
        plain.w["norm.bias"].zero_()
        assert rel_err(plain.logits(reqs["r1"]), ref["r1"]) > 1e-3
        plain.w["norm.bias"].copy_(saved)
        cuts = (traces.whole(reqs), traces.portions(reqs), traces.tail_one_by_one(reqs, 12), traces.mixed(reqs, {r: max(1, len(t) - 6) for r, t in reqs.items()}, max_live=3, seed=2))
        for dtype in ("float32", "bfloat16"):
            for graphs in (False, True):
                for steps in cuts:
                    steps = traces.last_only(steps) if graphs else steps
                    outs, _ = run_trace(folder, dtype, steps, max_live=3, cuda_graphs=graphs)
                    check(steps, outs, ref, TOL[dtype])
    finally:
        unregister_architecture("ToyParallelForCausalLM")
