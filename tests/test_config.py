"""Configuration: keys, defaults and rejections of the reference's Qwen3Config::Load
(src/model/causal_lm/qwen3_config.cpp:16-102), the registry rules of ResolveModelLoader
(src/model/loader.cpp:17-87), and the model spec built from a configuration."""

import json

import pytest

from tiny_configs import TINY, tiny_config
from zephyr_b200.config import (ConfigError, LayerCall, ModelSpec, Qwen3Config, load_model_config,
                                register_architecture, registered_architectures, resolve_architecture,
                                unregister_architecture)

BASE = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "vocab_size": 311,
    "hidden_size": 96, "intermediate_size": 200, "num_hidden_layers": 3, "num_attention_heads": 6,
    "num_key_value_heads": 3, "max_position_embeddings": 256, "rms_norm_eps": 1e-5,
}


def test_defaults_follow_the_reference():
    config = Qwen3Config.from_dict(BASE)
    assert config.head_dim == 96 // 6                 # absent head_dim -> hidden / heads
    assert config.rope_theta == 1000000.0 and config.tie_word_embeddings is False
    assert config.eos_token_ids == ()
    assert Qwen3Config.from_dict({**BASE, "head_dim": None}).head_dim == 16
    assert Qwen3Config.from_dict({**BASE, "head_dim": 32}).head_dim == 32   # heads*head_dim != hidden is fine


@pytest.mark.parametrize("key", ["hidden_act", "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
                                 "rms_norm_eps"])
def test_required_keys(key):
    config = dict(BASE)
    del config[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(config)


@pytest.mark.parametrize("patch,message", [
    ({"model_type": "llama"}, "dense Qwen3"),
    ({"quantization_config": {"bits": 4}}, "quantized"),
    ({"hidden_act": "gelu"}, "SiLU"),
    ({"attention_bias": True}, "bias-free"),
    ({"hidden_size": 96.0}, "int64 integer"),
    ({"vocab_size": True}, "int64 integer"),
    ({"num_hidden_layers": 2**70}, "int64 integer"),
    ({"num_key_value_heads": 4}, "divisible"),
    ({"head_dim": 15}, "even head width"),
    ({"rms_norm_eps": 0.0}, "finite positive"),
    ({"rope_theta": -1.0}, "finite positive"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "unscaled rotary"),
    ({"rope_scaling": {"type": "default", "partial_rotary_factor": 0.5}}, "unscaled rotary"),
    ({"rope_parameters": [1]}, "JSON object"),
    ({"layer_types": ["full_attention"]}, "every decoder layer"),
    ({"layer_types": ["full_attention", "linear_attention", "full_attention"]}, "only full-attention"),
    ({"layer_types": ["full_attention", "sliding_attention", "full_attention"], "sliding_window": 8}, "only full-attention"),
    ({"use_sliding_window": True, "sliding_window": 24}, "sliding-window attention is unsupported"),
    ({"use_sliding_window": True, "sliding_window": 24, "max_window_layers": 2}, "sliding-window attention is unsupported"),
    ({"eos_token_id": 400}, "outside the vocabulary"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"tie_word_embeddings": 1}, "true or false"),
])
def test_rejections(patch, message):
    with pytest.raises(ConfigError, match=message):
        Qwen3Config.from_dict({**BASE, **patch})


def test_rope_parameters_may_carry_theta():
    config = Qwen3Config.from_dict({**BASE, "rope_theta": 10.0,
                                    "rope_parameters": {"rope_type": "default", "rope_theta": 5000.0}})
    assert config.rope_theta == 5000.0
    assert Qwen3Config.from_dict({**BASE, "rope_scaling": None}).rope_theta == 1000000.0


def test_a_window_that_reaches_no_layer_is_accepted_as_the_reference_accepts_it():
    """qwen3_config.cpp:62-69: a configured window has no effect until it is enabled on a layer."""
    for patch in ({"use_sliding_window": True, "sliding_window": 24, "max_window_layers": 3},
                  {"use_sliding_window": False, "sliding_window": 24},
                  {"use_sliding_window": True, "sliding_window": None},
                  {"layer_types": ["full_attention"] * 3}):
        spec = Qwen3Config.from_dict({**BASE, **patch}).to_model_spec()
        assert all(layer.mixer.params["window"] == 0 for layer in spec.layers)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "W"])
def test_round_trip_and_spec(name, tmp_path):
    config = tiny_config(name)
    (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
    again = load_model_config(tmp_path)
    assert again == config
    spec = config.to_model_spec()
    assert isinstance(spec, ModelSpec) and len(spec.layers) == config.num_hidden_layers
    assert spec.run_order == tuple(LayerCall(i, i) for i in range(config.num_hidden_layers))
    assert (spec.output.params["weight"] == spec.input.params["weight"]) == config.tie_word_embeddings
    windows = TINY[name].get("windows", (0,) * config.num_hidden_layers)
    for index, layer in enumerate(spec.layers):
        p = layer.mixer.params
        assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["window"]) == (
            config.num_attention_heads, config.num_key_value_heads, config.head_dim, windows[index])
        assert set(layer.norms) == {"mixer", "feed_forward"}
        assert layer.norms["mixer"].eps == config.rms_norm_eps and layer.mixer.position.params["theta"] == config.rope_theta
        assert p["q_proj"] == f"model.layers.{index}.self_attn.q_proj.weight"


def test_the_two_tiny_configurations_differ_in_every_size():
    a, b = TINY["A"]["config"], TINY["B"]["config"]
    for key in a:
        assert a[key] != b[key], key
    assert TINY["A"]["page_size"] != TINY["B"]["page_size"]


def test_registry_rules():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture({"model_type": "qwen3"}).architecture == "Qwen3ForCausalLM"
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_class is Qwen3Config
    with pytest.raises(ConfigError, match="single architecture"):
        resolve_architecture({"architectures": ["Qwen3ForCausalLM", "X"]})
    with pytest.raises(ConfigError, match="unsupported"):
        resolve_architecture({"model_type": "qwen3", "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="unsupported"):
        resolve_architecture({})                       # neither identifier given
    with pytest.raises(ConfigError, match="unsupported"):
        resolve_architecture({"model_type": "llama", "architectures": ["Qwen3ForCausalLM"]})


def test_another_architecture_registers_without_touching_the_package():
    class ToyConfig:
        @classmethod
        def from_dict(cls, config, where="config.json"):
            return cls()

        def to_model_spec(self):
            return tiny_config("A").to_model_spec()

    register_architecture("toy", "ToyForCausalLM", ToyConfig)
    try:
        assert resolve_architecture({"model_type": "toy", "architectures": ["ToyForCausalLM"]}).config_class is ToyConfig
        with pytest.raises(ConfigError, match="already registered"):
            register_architecture("toy", "ToyForCausalLM", ToyConfig)
        with pytest.raises(ConfigError, match="lacks"):
            register_architecture("t2", "T2", object)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_run_order_validation():
    spec = tiny_config("A").to_model_spec()
    import dataclasses

    bad = dataclasses.replace(spec, run_order=(LayerCall(0, 0), LayerCall(1, 0)))
    with pytest.raises(ConfigError, match="written by"):
        bad.validate()
    bad = dataclasses.replace(spec, run_order=(LayerCall(0, 0, writes_cache=False),))
    with pytest.raises(ConfigError, match="before any call has written"):
        bad.validate()
    bad = dataclasses.replace(spec, run_order=(LayerCall(5, 0),))
    with pytest.raises(ConfigError, match="does not exist"):
        bad.validate()
    shared = dataclasses.replace(spec, run_order=(LayerCall(0, 0), LayerCall(1, 0, writes_cache=False), LayerCall(0, 1)))
    shared.validate()        # a layer named twice, and a layer reading another's cache
    assert shared.num_caches == 2


def test_missing_or_broken_file(tmp_path):
    with pytest.raises(ConfigError, match="cannot open"):
        load_model_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="invalid model configuration"):
        load_model_config(tmp_path)
