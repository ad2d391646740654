"""Typed configurations, the architecture registry, and the architecture-neutral model spec."""

from .errors import ConfigError, InvalidArgumentError, OutOfPagesError, WeightError, ZephyrError
from .qwen3 import Qwen3Config
from .registry import (ArchitectureEntry, load_model_config, load_model_spec, read_config_json,
                       register_architecture, registered_architectures, resolve_architecture,
                       unregister_architecture)
from .spec import (FeedForwardSpec, InputSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec, OutputSpec,
                   PositionSpec)

__all__ = [
    "ArchitectureEntry", "ConfigError", "FeedForwardSpec", "InputSpec", "InvalidArgumentError", "LayerCall", "LayerSpec",
    "MixerSpec", "ModelSpec", "NormSpec", "OutOfPagesError", "OutputSpec", "PositionSpec", "Qwen3Config", "WeightError",
    "ZephyrError", "load_model_config", "load_model_spec", "read_config_json", "register_architecture",
    "registered_architectures", "resolve_architecture", "unregister_architecture",
]
