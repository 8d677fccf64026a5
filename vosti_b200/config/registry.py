"""One registry from an architecture's name to the function that turns its
config.json into a `ModelSpec`.

The reference dispatches on a closed enum (src/model_config.rs:11-16,
src/exec/model.rs:205-621) keyed by its own family name; here the key is
``config.json: architectures[0]`` and the table is open.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Callable, Dict, Mapping

from .schema import ConfigError, ModelSpec

_ARCHITECTURES: Dict[str, Callable[[Mapping[str, Any]], ModelSpec]] = {}


def register_architecture(name: str, spec_from_config: Callable[[Mapping[str, Any]], ModelSpec],
                          *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = spec_from_config


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(raw: Mapping[str, Any]) -> str:
    names = raw.get("architectures") if isinstance(raw, Mapping) else None
    if not isinstance(names, list) or len(names) != 1 or not isinstance(names[0], str):
        raise ConfigError("config.json must name exactly one architecture in 'architectures'")
    return names[0]


def model_spec_from_config(raw: Mapping[str, Any]) -> ModelSpec:
    name = architecture_of(raw)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; known: {known_architectures()}")
    spec = _ARCHITECTURES[name](raw)
    spec.validate()
    return spec


def read_config_json(model_dir: str | Path) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path} is not valid JSON: {error}") from error


def model_spec_from_dir(model_dir: str | Path) -> ModelSpec:
    return model_spec_from_config(read_config_json(model_dir))
