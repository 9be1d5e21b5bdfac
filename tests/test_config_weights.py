"""Configuration from config.json keys, the architecture registry, and the loader's errors."""

from __future__ import annotations

import json

import pytest
import torch

from helpers import TINY, make_model_dir
from kvforge_b200 import PRESETS, ConfigError, EngineConfig, ModelConfig
from kvforge_b200.config.engine_config import CacheConfig, SchedulerConfig
from kvforge_b200.config.registry import ARCHITECTURES, architecture_of, get_architecture
from kvforge_b200.parts.model import DecoderModel
from kvforge_b200.weights.loader import WeightsError, load_weights
from kvforge_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def test_config_json_roundtrip_reads_every_key():
    for name, t in TINY.items():
        cfg = t["cfg"]
        d = json.loads(json.dumps(cfg.to_hf_dict()))
        back = ModelConfig.from_hf_dict(d)
        assert back == cfg, name
    d = PRESETS["tiny-b"].to_hf_dict()
    assert d["rope_scaling"]["rope_type"] == "llama3" and d["num_key_value_heads"] == 1


def test_config_defaults_follow_kvforge():
    d = dict(vocab_size=10, hidden_size=8, num_hidden_layers=1, num_attention_heads=2, intermediate_size=16,
             rms_norm_eps=1e-5, max_position_embeddings=64, eos_token_id=[7, 9])  # fmt: skip
    cfg = ModelConfig.from_hf_dict(d)
    assert cfg.num_kv_heads == 2 and cfg.head_dim == 4 and cfg.rope_theta == 10000.0
    assert cfg.eos_token_id == 7 and cfg.tie_word_embeddings is False and cfg.rope_scaling is None


@pytest.mark.parametrize(
    "patch",
    [
        {"attention_bias": True},
        {"mlp_bias": True},
        {"hidden_act": "gelu"},
        {"rope_scaling": {"rope_type": "yarn", "factor": 2.0}},
        {"rope_scaling": {"rope_type": "llama3", "factor": 2.0}},
        {"num_key_value_heads": 3},
        {"architectures": ["MambaForCausalLM"]},
    ],
)
def test_config_rejects_what_is_not_built(patch):
    d = PRESETS["tiny-a"].to_hf_dict()
    d.update(patch)
    with pytest.raises(ConfigError):
        architecture_of(d).parse_config(d)


def test_config_missing_key_is_named():
    d = PRESETS["tiny-a"].to_hf_dict()
    del d["rms_norm_eps"]
    with pytest.raises(ConfigError, match="rms_norm_eps"):
        ModelConfig.from_hf_dict(d)


def test_registry_maps_name_to_model():
    arch = get_architecture("LlamaForCausalLM")
    spec = arch.build_spec(PRESETS["tiny-b"])
    assert "LlamaForCausalLM" in ARCHITECTURES
    assert len(spec.layers) == 3 and [c.layer for c in spec.execution] == [0, 1, 2]
    mixer = spec.layers[0].block.params["mixer"]
    assert mixer.kind == "paged_attention" and mixer.params["num_kv_heads"] == 1
    assert mixer.params["position"].params["scaling"]["factor"] == 8.0


def test_engine_config_clamps_and_follows_dtype():
    ec = EngineConfig(model=PRESETS["tiny-a"], cache=CacheConfig(), scheduler=SchedulerConfig(max_model_len=4096), dtype="float32")
    assert ec.scheduler.max_model_len == 128 and ec.cache.dtype == torch.float32
    with pytest.raises(ValueError):
        EngineConfig(model=PRESETS["tiny-a"], dtype="float16")
    assert CacheConfig(num_blocks=None, kv_cache_memory_gb=1.0).resolve_num_blocks(1 << 20) == 1024


def test_expected_weight_names_are_kvforge_parameter_names():
    model = DecoderModel(get_architecture("LlamaForCausalLM").build_spec(PRESETS["tiny-a"]))
    names = set(model.expected_weights())
    per_layer = {"input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                 "self_attn.o_proj.weight", "post_attention_layernorm.weight", "mlp.gate_proj.weight",
                 "mlp.up_proj.weight", "mlp.down_proj.weight"}  # fmt: skip
    want = {"model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"}
    want |= {f"model.layers.{i}.{n}" for i in range(2) for n in per_layer}
    assert names == want


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(4)}
    write_safetensors(tmp_path / "x.safetensors", t)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.keys()) == ["a", "b", "c"]
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v) and f.info(k) == (v.dtype, tuple(v.shape))


def test_loader_reports_missing_unexpected_and_shapes_in_one_error(tmp_path):
    d = make_model_dir(tmp_path, "tiny-b")
    model = DecoderModel(get_architecture("LlamaForCausalLM").build_spec(TINY["tiny-b"]["cfg"]))
    expected = model.expected_weights()
    ok = load_weights(d, expected, torch.float32, "cpu")
    assert ok["model.norm.weight"].dtype == torch.float32
    f = SafetensorsFile(d / "model.safetensors")
    tensors = {k: f.tensor(k).clone() for k in f.keys()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(96)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 96)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)  # ignored, as in kvforge
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text((d / "config.json").read_text())
    write_safetensors(bad / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as e:
        load_weights(bad, expected, torch.float32, "cpu", ignore_suffixes=("rotary_emb.inv_freq",))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(err.wrong_shape) == 1 and "k_proj" in err.wrong_shape[0] and "[32, 96]" in err.wrong_shape[0]
    msg = str(err)
    assert "missing" in msg and "unexpected" in msg and "wrong shape" in msg


def test_loader_storage_rules(tmp_path):
    # matrices follow the engine's storage type; vectors are held in float32 whatever the file has
    d = make_model_dir(tmp_path, "tiny-a", store_dtype=torch.bfloat16)
    model = DecoderModel(get_architecture("LlamaForCausalLM").build_spec(TINY["tiny-a"]["cfg"]))
    w = load_weights(d, model.expected_weights(), torch.bfloat16, "cpu")
    assert w["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert w["model.layers.0.input_layernorm.weight"].dtype == torch.float32
    assert "lm_head.weight" not in w  # tied: the folder has no separate head
    w32 = load_weights(d, model.expected_weights(), torch.float32, "cpu")
    assert torch.equal(w32["model.embed_tokens.weight"], w["model.embed_tokens.weight"].float())


def test_a_checkpoint_in_shards_reads_like_one_file(tmp_path):
    """The same tensors split over two files with an index (the layout of larger checkpoints),
    and the same two files without an index: both load to what the single file gives."""
    import json

    d = make_model_dir(tmp_path, "tiny-b")
    model = DecoderModel(get_architecture("LlamaForCausalLM").build_spec(TINY["tiny-b"]["cfg"]))
    expected = model.expected_weights()
    one = load_weights(d, expected, torch.float32, "cpu")
    f = SafetensorsFile(d / "model.safetensors")
    names = sorted(f.keys())
    halves = (names[::2], names[1::2])
    for with_index in (True, False):
        sharded = tmp_path / f"sharded-{with_index}"
        sharded.mkdir()
        (sharded / "config.json").write_text((d / "config.json").read_text())
        weight_map = {}
        for i, part in enumerate(halves):
            fname = f"model-{i + 1:05d}-of-00002.safetensors"
            write_safetensors(sharded / fname, {n: f.tensor(n).clone() for n in part})
            weight_map.update({n: fname for n in part})
        if with_index:
            (sharded / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
        got = load_weights(sharded, expected, torch.float32, "cpu")
        assert sorted(got) == sorted(one) and all(torch.equal(got[n], one[n]) for n in one)
    # a shard that is missing shows as its tensors missing, in the one error
    (tmp_path / "sharded-False" / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(WeightsError) as e:
        load_weights(tmp_path / "sharded-False", expected, torch.float32, "cpu")
    assert sorted(e.value.missing) == sorted(n for n in halves[1] if not expected[n].optional)


def test_bytes_as_tokens_fit_the_vocabulary():
    from kvforge_b200.engine.tokenizer import BytesAsTokens

    big = BytesAsTokens(320)
    ids = big.encode("héllo")
    assert ids[0] == 256 and ids[1:] == list("héllo".encode()) and big.eos_token_id == 257
    assert big.decode(ids + [257]) == "héllo"
    exact = BytesAsTokens(256)  # no room for the two marks
    assert exact.encode("hi") == [104, 105] and exact.eos_token_id is None and exact.bos_token_id is None
    small = BytesAsTokens(200)
    assert all(0 <= t < 200 for t in small.encode("héllo ÿ"))
