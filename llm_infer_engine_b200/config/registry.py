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


def _id_list(value, where: str):
    if value is None:
        return []
    ids = [value] if isinstance(value, int) and not isinstance(value, bool) else value
    if not isinstance(ids, (list, tuple)) or not all(isinstance(e, int) and not isinstance(e, bool) for e in ids):
        raise ConfigError(f"{where}: eos_token_id must be an integer or a list of integers, got {value!r}")
    return list(ids)


def merge_generation_config(config_json: dict, model_dir: str) -> dict:
    """Checkpoints keep the ids at which generation stops in two places: `eos_token_id` of config.json and of
    generation_config.json (often a longer list there). Both are taken: the union, config.json's first."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return config_json
    try:
        with open(path, "r", encoding="utf-8") as f:
            gen = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(gen, dict):
        raise ConfigError(f"{path}: top level must be an object")
    ids = _id_list(config_json.get("eos_token_id"), "config.json")
    ids += [e for e in _id_list(gen.get("eos_token_id"), "generation_config.json") if e not in ids]
    if ids:
        config_json = dict(config_json, eos_token_id=ids if len(ids) > 1 else ids[0])
    return config_json


def load_config(source):
    """`source` is a model folder (config.json, and generation_config.json for further stop ids if it is
    there) or an already parsed config.json dict. Returns (architecture, typed config)."""
    if isinstance(source, (str, os.PathLike)):
        config_json = merge_generation_config(read_config_json(source), source)
    else:
        config_json = dict(source)
    arch = architecture_of(config_json)
    return arch, arch.config_cls.from_dict(config_json)
