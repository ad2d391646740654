"""The configurations of the tests.

A and B are the two tiny ones the benchmark description names; they differ in every size and
option.  D, E and F are small in depth and vocabulary but have the head size and the layer widths of
the benchmarked models, so that whole-model tests run the kernels those models run: D is the
smallest model with head size 128 (tensor-core prompt attention, the fast decode attention), E has
two layers of the 0.6B widths (the fused chain of a decode layer at its benchmarked shape), F one
layer of the 8B widths (rows longer than 1024 in the chain, and a down projection whose input does
not fit beside the weight ring in shared memory).  L is one small layer of head size 128 whose position table
reaches 4608, for contexts as long as the benchmark's.

C and W are NOT Qwen3: they belong to a test-only architecture, ``TinyWindowedForCausalLM``, defined
and registered here, which is the Qwen3 decoder with a sliding window on some layers (the reference
rejects such a configuration, src/model/causal_lm/qwen3_config.cpp:63-80; the attention part and the
cache manager take a window as a parameter).  C adds a group of four query heads per key/value head
and a head size (48) that only the general attention kernel takes; W has head size 64, which the
fast decode and prompt kernels take, so that window release and reused pages meet those kernels.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass

from zephyr_b200.config import ConfigError, Qwen3Config, register_architecture, registered_architectures

TINY = {
    "A": dict(seed=0, page_size=4, config=dict(
        vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=10000.0,
        tie_word_embeddings=True)),
    "B": dict(seed=1, page_size=8, config=dict(
        vocab_size=311, hidden_size=96, intermediate_size=200, num_hidden_layers=3, num_attention_heads=6,
        num_key_value_heads=3, head_dim=32, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=1000000.0,
        tie_word_embeddings=False)),
    "C": dict(seed=2, page_size=16, windows=(0, 24, 24), config=dict(
        vocab_size=199, hidden_size=80, intermediate_size=144, num_hidden_layers=3, num_attention_heads=8,
        num_key_value_heads=2, head_dim=48, max_position_embeddings=256, rms_norm_eps=3e-6, rope_theta=500000.0,
        tie_word_embeddings=False)),
    "W": dict(seed=6, page_size=8, windows=(24, 0, 40), config=dict(
        vocab_size=173, hidden_size=112, intermediate_size=168, num_hidden_layers=3, num_attention_heads=4,
        num_key_value_heads=2, head_dim=64, max_position_embeddings=512, rms_norm_eps=2e-6, rope_theta=30000.0,
        tie_word_embeddings=True)),
    "D": dict(seed=3, page_size=16, config=dict(
        vocab_size=503, hidden_size=256, intermediate_size=520, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=128, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=1000000.0,
        tie_word_embeddings=False)),
    "E": dict(seed=4, page_size=16, config=dict(
        vocab_size=1001, hidden_size=1024, intermediate_size=3072, num_hidden_layers=2, num_attention_heads=16,
        num_key_value_heads=8, head_dim=128, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=1000000.0,
        tie_word_embeddings=True)),
    "L": dict(seed=8, page_size=16, config=dict(       # one small layer with head size 128 and room for long contexts
        vocab_size=331, hidden_size=128, intermediate_size=264, num_hidden_layers=1, num_attention_heads=2,
        num_key_value_heads=1, head_dim=128, max_position_embeddings=4608, rms_norm_eps=1e-6, rope_theta=1000000.0,
        tie_word_embeddings=True)),
    "F": dict(seed=5, page_size=16, config=dict(
        vocab_size=517, hidden_size=4096, intermediate_size=12288, num_hidden_layers=1, num_attention_heads=32,
        num_key_value_heads=8, head_dim=128, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=1000000.0,
        tie_word_embeddings=False)),
}


@dataclass(frozen=True)
class TinyWindowedConfig:
    """The Qwen3 decoder with ``layer_windows[i]`` positions visible in layer i (0 = all).  Its
    config.json is Qwen3's with another ``model_type`` and ``architectures`` and the extra key."""

    base: Qwen3Config
    layer_windows: tuple[int, ...]

    architecture = "TinyWindowedForCausalLM"
    model_type = "tiny_windowed"

    def __getattr__(self, name):            # sizes are read off the base configuration
        return getattr(object.__getattribute__(self, "base"), name)

    @classmethod
    def from_dict(cls, config, where="config.json"):
        windows = config.get("layer_windows")
        if not isinstance(windows, list) or any(not isinstance(w, int) or w < 0 for w in windows):
            raise ConfigError(f"{where}: 'layer_windows' must be a list of non-negative integers")
        plain = {k: v for k, v in config.items() if k not in ("layer_windows", "model_type", "architectures")}
        base = Qwen3Config.from_dict({**plain, "model_type": "qwen3"}, where)
        if len(windows) != base.num_hidden_layers:
            raise ConfigError(f"{where}: 'layer_windows' must have one entry per layer")
        return cls(base, tuple(windows))

    def to_dict(self):
        return {**self.base.to_dict(), "model_type": self.model_type, "architectures": [self.architecture],
                "layer_windows": list(self.layer_windows)}

    def to_model_spec(self):
        spec = self.base.to_model_spec()
        layers = tuple(
            dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, params={**layer.mixer.params, "window": w}))
            for layer, w in zip(spec.layers, self.layer_windows))
        return dataclasses.replace(spec, architecture=self.architecture, layers=layers)


if TinyWindowedConfig.architecture not in registered_architectures():
    register_architecture(TinyWindowedConfig.model_type, TinyWindowedConfig.architecture, TinyWindowedConfig)


def tiny_config(name: str):
    base = Qwen3Config(**TINY[name]["config"])
    if "windows" in TINY[name]:
        return TinyWindowedConfig(base, tuple(TINY[name]["windows"]))
    return base
