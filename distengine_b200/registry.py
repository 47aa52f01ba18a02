"""One registry from the architecture's name (config.json ``architectures[0]``) to its model.

An entry holds the typed configuration's parser and the function that builds the model from it.
The reference has no registry: it constructs ``LlamaForCausalLM`` directly
(src/utils/load_model.py:17, src/distengine/worker.py:414).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .config.model import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], ModelConfig]
    build_model: Callable[..., Any]          # (config, dtype, device) -> model without weights


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable[[Mapping[str, Any]], ModelConfig],
                          build_model: Callable[..., Any]) -> None:
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_model)


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    from . import models  # noqa: F401  (registers the built-in architectures on import)


def resolve(config_json: Mapping[str, Any]) -> tuple[Architecture, ModelConfig]:
    """The architecture entry and the parsed configuration for a config.json."""
    _ensure_builtin()
    names = config_json.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json: key 'architectures' must be a list with the model "
                          "class's name")
    name = names[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"config.json: architecture '{name}' is not registered; known: "
                          f"{', '.join(sorted(_ARCHITECTURES))}")
    entry = _ARCHITECTURES[name]
    return entry, entry.parse_config(config_json)


def read_config(model_dir: str) -> tuple[Architecture, ModelConfig]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path}: a model folder holds config.json and model.safetensors")
    with open(path) as handle:
        return resolve(json.load(handle))
