"""Configuration and registry (no GPU)."""
import json

import pytest

from helpers import TINY, tiny_config, tiny_config_dict
from tinyserve_b200.config import (ConfigError, EngineConfig, ModelConfig, Qwen3Config,
                                   config_from_dict, load_model_config, register_architecture)
from tinyserve_b200.config.registry import ARCHITECTURES
from tinyserve_b200.parts import build_model


@pytest.mark.parametrize("name", sorted(TINY))
def test_every_size_comes_from_config(name):
    raw = tiny_config_dict(name)
    cfg = config_from_dict(raw)
    assert isinstance(cfg, Qwen3Config)
    for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "intermediate_size", "rms_norm_eps", "rope_theta",
                "tie_word_embeddings"):
        assert getattr(cfg, key) == raw[key]
    spec = cfg.model_spec()
    assert len(spec.layers) == raw["num_hidden_layers"]
    m = spec.layers[0].mixer
    assert m.get("head_dim") == raw["head_dim"] and m.get("num_kv_heads") == raw["num_key_value_heads"]
    assert m.get("scale") == raw["head_dim"] ** -0.5
    assert spec.layers[0].ffn.get("intermediate_size") == raw["intermediate_size"]
    assert spec.final_norm.get("eps") == raw["rms_norm_eps"]


def test_round_trip_and_folder(tmp_path):
    cfg = tiny_config("C")
    again = config_from_dict(cfg.to_dict())
    assert again == cfg
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_model_config(str(tmp_path)) == cfg


def test_defaults_follow_the_reference():
    raw = tiny_config_dict("A")
    del raw["head_dim"], raw["tie_word_embeddings"], raw["rope_theta"], raw["num_key_value_heads"]
    cfg = config_from_dict(raw)
    assert cfg.head_dim == raw["hidden_size"] // raw["num_attention_heads"]   # serve.py:821
    assert cfg.tie_word_embeddings is False                                   # serve.py:1209
    assert cfg.rope_theta == 10000.0                                          # serve.py:1222
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    raw["rope_parameters"] = {"rope_type": "default", "rope_theta": 123.0}
    assert config_from_dict(raw).rope_theta == 123.0                          # serve.py:1219-1222


@pytest.mark.parametrize("change, message", [
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"rope_type": "yarn"}}, "rope_type"),
    ({"architectures": ["NopeForCausalLM"]}, "not registered"),
    ({"architectures": None}, "architectures"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"vocab_size": "many"}, "integer"),
])
def test_bad_configs_are_refused(change, message):
    raw = dict(tiny_config_dict("A"), **change)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_window_layers():
    cfg = tiny_config("C")
    assert [cfg.layer_window(i) for i in range(4)] == [0, 0, 40, 40]
    raw = dict(tiny_config_dict("C"), layer_types=["sliding_attention", "full_attention"] * 2)
    cfg = config_from_dict(raw)
    assert [cfg.layer_window(i) for i in range(4)] == [40, 0, 40, 0]
    model = build_model(cfg)
    assert [g.kind for g in model.cache_groups] == ["window", "full"]
    assert model.group_sizes == [2, 2]
    off = config_from_dict(dict(tiny_config_dict("C"), use_sliding_window=False))
    assert [off.layer_window(i) for i in range(4)] == [0] * 4


def test_registering_another_architecture():
    class OtherConfig(Qwen3Config):
        architecture = "OtherForCausalLM"

        @classmethod
        def from_dict(cls, raw):
            return super().from_dict(dict(raw, model_type="qwen3"))

    register_architecture("OtherForCausalLM", OtherConfig)
    try:
        cfg = config_from_dict(dict(tiny_config_dict("A"), architectures=["OtherForCausalLM"]))
        assert type(cfg) is OtherConfig
    finally:
        ARCHITECTURES.pop("OtherForCausalLM")
    with pytest.raises(TypeError):
        register_architecture("X", dict)


def test_engine_config_checks():
    assert EngineConfig(model="m", dtype="bf16").dtype == "bfloat16"
    assert EngineConfig(model="m", dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError):
        EngineConfig(model="m", dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(model="m", block_size=12)


def test_run_order_is_data():
    from tinyserve_b200.config import LayerCall, ModelSpec
    from tinyserve_b200.parts import DecoderModel
    spec = tiny_config("A").model_spec()
    # layer 0 runs twice (own caches), then layer 1 reads the cache that the first call wrote
    order = (LayerCall(0, 0), LayerCall(0, 1), LayerCall(1, 0, writes_cache=False))
    model = DecoderModel(ModelSpec(spec.vocab_size, spec.hidden_size, spec.layers, order,
                                   spec.final_norm, spec.tie_word_embeddings))
    assert [(c.layer, c.cache, c.writes_cache) for c in model.calls] == \
        [(0, 0, True), (0, 1, True), (1, 0, False)]
    assert model.group_sizes == [2]
    with pytest.raises(ValueError, match="never written"):
        DecoderModel(ModelSpec(spec.vocab_size, spec.hidden_size, spec.layers,
                               (LayerCall(0, 0, writes_cache=False),), spec.final_norm, True))
    with pytest.raises(ValueError, match="two calls"):
        DecoderModel(ModelSpec(spec.vocab_size, spec.hidden_size, spec.layers,
                               (LayerCall(0, 0), LayerCall(1, 0)), spec.final_norm, True))
