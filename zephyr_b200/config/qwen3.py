"""Typed configuration of the dense Qwen3 decoder, read from config.json.

Keys, defaults and rejections follow the reference's
``Qwen3Config::Load`` (src/model/causal_lm/qwen3_config.cpp:16-102) and the
validation in ``Qwen3Model::Load`` (src/model/causal_lm/qwen3.cpp:102-112).
Every layer is full causal attention: a sliding window that would reach a
layer, and any ``layer_types`` entry other than ``"full_attention"``, are
rejected as the reference rejects them (qwen3_config.cpp:63-80).  (The
attention part and the cache manager do take a window as a parameter; no
key of this architecture's config.json sets it.)
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError
from .spec import (FeedForwardSpec, InputSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec, OutputSpec,
                   PositionSpec)

_INT64_MAX = 2**63 - 1


def _read_dimension(config: Mapping[str, Any], name: str) -> int:
    """An integer JSON number within int64 (qwen3_config.cpp:35-44); bools and floats are refused."""
    if name not in config:
        raise ConfigError(f"Qwen3 configuration lacks the required key '{name}'")
    value = config[name]
    if isinstance(value, bool) or not isinstance(value, int) or not -_INT64_MAX - 1 <= value <= _INT64_MAX:
        raise ConfigError(f"Qwen3 configuration field '{name}' must be an int64 integer, got {value!r}")
    return value


def _read_number(config: Mapping[str, Any], name: str, default: float | None = None) -> float:
    if name not in config:
        if default is None:
            raise ConfigError(f"Qwen3 configuration lacks the required key '{name}'")
        return default
    value = config[name]
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"Qwen3 configuration field '{name}' must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    tie_word_embeddings: bool = False
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, config: Mapping[str, Any], where: str = "config.json") -> "Qwen3Config":
        if not isinstance(config, Mapping):
            raise ConfigError(f"{where}: the configuration must be a JSON object")
        if config.get("model_type", "qwen3") != "qwen3":
            raise ConfigError(f"{where}: Qwen3Config requires a dense Qwen3 model (model_type 'qwen3')")
        if config.get("quantization_config") is not None:
            raise ConfigError(f"{where}: quantized Qwen3 checkpoints are unsupported")
        if "hidden_act" not in config:
            raise ConfigError(f"{where}: Qwen3 configuration lacks the required key 'hidden_act'")
        if config["hidden_act"] != "silu" or config.get("attention_bias", False):
            raise ConfigError(f"{where}: Qwen3 requires SiLU activation and bias-free attention projections")

        vocab = _read_dimension(config, "vocab_size")
        hidden = _read_dimension(config, "hidden_size")
        inter = _read_dimension(config, "intermediate_size")
        layers = _read_dimension(config, "num_hidden_layers")
        heads = _read_dimension(config, "num_attention_heads")
        kv_heads = _read_dimension(config, "num_key_value_heads")
        max_pos = _read_dimension(config, "max_position_embeddings")
        if config.get("head_dim") is not None:
            head_dim = _read_dimension(config, "head_dim")
        else:
            head_dim = hidden // heads if heads > 0 else 0
        eps = _read_number(config, "rms_norm_eps")
        theta = _read_number(config, "rope_theta", 1000000.0)
        tied = config.get("tie_word_embeddings", False)
        if not isinstance(tied, bool):
            raise ConfigError(f"{where}: 'tie_word_embeddings' must be true or false")

        # Both checkpoint schemas may describe ordinary RoPE (qwen3_config.cpp:83-97).
        for key in ("rope_scaling", "rope_parameters"):
            rope = config.get(key)
            if rope is None:
                continue
            if not isinstance(rope, Mapping):
                raise ConfigError(f"{where}: '{key}' must be a JSON object")
            rope_type = rope.get("rope_type", rope.get("type"))
            if rope_type is None:
                raise ConfigError(f"{where}: '{key}' lacks 'rope_type'")
            if rope_type != "default" or float(rope.get("partial_rotary_factor", 1.0)) != 1.0:
                raise ConfigError(f"{where}: only full-head, unscaled rotary embeddings are supported")
            theta = _read_number(rope, "rope_theta", theta)

        cls._reject_windows(config, layers, where)

        eos = config.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"{where}: 'eos_token_id' must be an integer or a list of integers")

        result = cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                     num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                     max_position_embeddings=max_pos, rms_norm_eps=eps, rope_theta=theta,
                     tie_word_embeddings=tied, eos_token_ids=eos_ids)
        result.validate(where)
        return result

    @staticmethod
    def _reject_windows(config: Mapping[str, Any], layers: int, where: str) -> None:
        """qwen3_config.cpp:62-80: a configured window has no effect until it is enabled on at least one
        decoder layer (``max_window_layers`` below the layer count), and then it is refused; so is a
        ``layer_types`` list that is not ``layers`` times "full_attention"."""
        if config.get("use_sliding_window", False) and config.get("sliding_window") is not None:
            first = _read_dimension(config, "max_window_layers") if "max_window_layers" in config else 0
            if first < layers:
                raise ConfigError(f"{where}: Qwen3 sliding-window attention is unsupported")
        layer_types = config.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != layers:
                raise ConfigError(f"{where}: Qwen3 layer_types must describe every decoder layer")
            if any(kind != "full_attention" for kind in layer_types):
                raise ConfigError(f"{where}: Qwen3 supports only full-attention decoder layers")

    @classmethod
    def from_file(cls, path: str | Path) -> "Qwen3Config":
        path = Path(path)
        try:
            text = path.read_text(encoding="utf-8")
        except OSError as error:
            raise ConfigError(f"cannot open Qwen3 configuration: {path} ({error.strerror})") from error
        try:
            data = json.loads(text)
        except json.JSONDecodeError as error:
            raise ConfigError(f"{path}: invalid Qwen3 configuration: {error}") from error
        return cls.from_dict(data, str(path))

    # --------------------------------------------------------------- validation
    def validate(self, where: str = "config") -> None:
        """The checks of Qwen3Model::Load (qwen3.cpp:102-112)."""
        dims = (self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers,
                self.num_attention_heads, self.num_key_value_heads, self.head_dim, self.max_position_embeddings)
        if (any(d <= 0 for d in dims) or self.head_dim % 2 != 0
                or self.num_attention_heads % self.num_key_value_heads != 0
                or not math.isfinite(self.rms_norm_eps) or self.rms_norm_eps <= 0.0
                or not math.isfinite(self.rope_theta) or self.rope_theta <= 0.0):
            raise ConfigError(
                f"{where}: Qwen3 requires positive dimensions, divisible Q/KV heads, an even head width, "
                "and finite positive normalization/rotary parameters")
        for token in self.eos_token_ids:
            if not 0 <= token < self.vocab_size:
                raise ConfigError(f"{where}: eos token id {token} lies outside the vocabulary")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        """config.json content that ``from_dict`` reads back to an equal configuration."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_act": "silu",
            "attention_bias": False,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        out["use_sliding_window"] = False
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return out

    # --------------------------------------------------------------- model spec
    def to_model_spec(self) -> ModelSpec:
        """The parts of the model, layer by layer, with the tensor names the reference reads
        (qwen3.cpp:21-31,73-77,121-136; mlp.cpp:21-25)."""
        position = PositionSpec(kind="rope_neox", head_dim=self.head_dim,
                                max_positions=self.max_position_embeddings, params={"theta": self.rope_theta})
        layers = []
        for index in range(self.num_hidden_layers):
            prefix = f"model.layers.{index}"
            mixer = MixerSpec(kind="attention", position=position, params={
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "window": 0,
                "qk_norm_eps": self.rms_norm_eps,
                "q_proj": f"{prefix}.self_attn.q_proj.weight",
                "k_proj": f"{prefix}.self_attn.k_proj.weight",
                "v_proj": f"{prefix}.self_attn.v_proj.weight",
                "o_proj": f"{prefix}.self_attn.o_proj.weight",
                "q_norm": f"{prefix}.self_attn.q_norm.weight",
                "k_norm": f"{prefix}.self_attn.k_norm.weight",
            })
            ffn = FeedForwardSpec(kind="swiglu", params={
                "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size,
                "gate_proj": f"{prefix}.mlp.gate_proj.weight",
                "up_proj": f"{prefix}.mlp.up_proj.weight",
                "down_proj": f"{prefix}.mlp.down_proj.weight",
            })
            layers.append(LayerSpec(
                block="prenorm_residual", mixer=mixer, feed_forward=ffn,
                norms={"mixer": NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps,
                                         f"{prefix}.input_layernorm.weight"),
                       "feed_forward": NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps,
                                                f"{prefix}.post_attention_layernorm.weight")}))
        embedding = "model.embed_tokens.weight"
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_seq_len=self.max_position_embeddings,
            input=InputSpec("embedding", {"weight": embedding, "vocab_size": self.vocab_size,
                                          "hidden_size": self.hidden_size}),
            layers=tuple(layers),
            run_order=tuple(LayerCall(layer=i, cache=i) for i in range(self.num_hidden_layers)),
            # A tied head reads the embedding table itself: the same tensor name (qwen3.cpp:134-136).
            output=OutputSpec("norm_head", {
                "norm": NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps, "model.norm.weight"),
                "weight": embedding if self.tie_word_embeddings else "lm_head.weight",
                "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            eos_token_ids=self.eos_token_ids,
            # A tied checkpoint may still carry a copy of the head; the reference never reads it (qwen3.cpp:134).
            ignorable_weights=("lm_head.weight",) if self.tie_word_embeddings else (),
        )
        spec.validate()
        return spec
