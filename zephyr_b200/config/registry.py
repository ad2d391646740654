"""One registry from an architecture's name to its configuration class.

A configuration class offers ``from_dict(config, where)`` and
``to_model_spec()``; the spec names the parts, and ``parts.build_model``
builds the model from it.  The matching rules are those of the reference's
``ResolveModelLoader`` (src/model/loader.cpp:17-87): every identifier the
file supplies must select the same entry; at most one architecture may be
named; no match and several matches are both errors.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError
from .qwen3 import Qwen3Config
from .spec import ModelSpec


@dataclass(frozen=True)
class ArchitectureEntry:
    model_type: str
    architecture: str
    config_class: Any


_ARCHITECTURES: dict[str, ArchitectureEntry] = {}


def register_architecture(model_type: str, architecture: str, config_class: Any) -> None:
    """Add an architecture.  ``config_class`` needs ``from_dict`` and ``to_model_spec``."""
    if architecture in _ARCHITECTURES:
        raise ConfigError(f"architecture '{architecture}' is already registered")
    for method in ("from_dict", "to_model_spec"):
        if not hasattr(config_class, method):
            raise ConfigError(f"configuration class for '{architecture}' lacks {method}()")
    _ARCHITECTURES[architecture] = ArchitectureEntry(model_type, architecture, config_class)


def unregister_architecture(architecture: str) -> None:
    _ARCHITECTURES.pop(architecture, None)


def registered_architectures() -> tuple[str, ...]:
    return tuple(_ARCHITECTURES)


def resolve_architecture(config: Mapping[str, Any], where: str = "config.json") -> ArchitectureEntry:
    if not isinstance(config, Mapping):
        raise ConfigError(f"{where}: the configuration must be a JSON object")
    has_model_type = "model_type" in config
    model_type = config.get("model_type", "")
    architectures = config.get("architectures") or []
    if not isinstance(architectures, list) or any(not isinstance(a, str) for a in architectures):
        raise ConfigError(f"{where}: 'architectures' must be a list of strings")
    if len(architectures) > 1:
        raise ConfigError(f"{where}: the configuration must select a single architecture")
    selected = None
    for entry in _ARCHITECTURES.values():
        matches_type = (model_type == entry.model_type) if has_model_type else bool(architectures)
        matches_arch = not architectures or architectures[0] == entry.architecture
        if not (matches_type and matches_arch):
            continue
        if selected is not None:
            raise ConfigError(f"{where}: ambiguous model configuration; name the architecture")
        selected = entry
    if selected is None:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise ConfigError(
            f"{where}: unsupported model configuration (model_type={model_type!r}, "
            f"architectures={architectures!r}); registered architectures: {known}")
    return selected


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    try:
        text = path.read_text(encoding="utf-8")
    except OSError as error:
        raise ConfigError(f"cannot open model configuration: {path} ({error.strerror})") from error
    try:
        data = json.loads(text)
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path}: invalid model configuration: {error}") from error
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: the configuration must be a JSON object")
    return data


def load_model_config(model_dir: str | Path):
    """Read ``model_dir/config.json`` and return the typed configuration its architecture names."""
    data = read_config_json(model_dir)
    where = str(Path(model_dir) / "config.json")
    entry = resolve_architecture(data, where)
    return entry.config_class.from_dict(data, where)


def load_model_spec(model_dir: str | Path) -> ModelSpec:
    return load_model_config(model_dir).to_model_spec()


register_architecture(Qwen3Config.model_type, Qwen3Config.architecture, Qwen3Config)
