"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

An architecture registers a typed configuration class with a `from_dict(config_json)`
constructor and a `to_spec(config) -> ModelSpec` function. Everything downstream (weights,
cache, step, generation, replay) works from the `ModelSpec`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .spec import ModelSpec


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any
    to_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Any, to_spec: Callable[[Any], ModelSpec]) -> None:
    if not hasattr(config_cls, "from_dict"):
        raise TypeError(f"{config_cls!r} needs a from_dict(config_json) constructor")
    _ARCHITECTURES[name] = Architecture(name, config_cls, to_spec)


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_of(config_json: dict) -> Architecture:
    archs = config_json.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names; "
                          f"known architectures: {known_architectures()}")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"config.json: unknown architecture {name!r}; known architectures: "
                          f"{known_architectures()}")
    return _ARCHITECTURES[name]


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    try:
        with open(path, "r", encoding="utf-8") as f:
            data = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return data


def load_config(source):
    """`source` is a model folder or an already parsed config.json dict.
    Returns (architecture, typed config)."""
    config_json = read_config_json(source) if isinstance(source, (str, os.PathLike)) else dict(source)
    arch = architecture_of(config_json)
    return arch, arch.config_cls.from_dict(config_json)
