"""Typed model configurations and the one registry from architecture name to model.

The reference has no registry: it tests ``model_type`` against a string and
constructs its only model class directly (model/src/qwen3_checkpoint.cpp:30-33,
model/model_main.cpp:577).  Here every architecture registers three things under
the name that ``config.json`` carries in ``architectures[0]``: its typed
configuration class, a function that turns a configuration into a model
description (layer specs and their order), and nothing else; the engine, the
cache, the scheduler and the tools only ever go through this registry.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, Type


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration."""


class ModelConfig:
    """Base of the typed configurations.  A subclass is a dataclass that holds every
    number its architecture needs; nothing in the framework carries a size or a
    constant that config.json gives."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":  # pragma: no cover - interface
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:  # pragma: no cover - interface
        raise NotImplementedError

    def validate(self) -> None:  # pragma: no cover - interface
        raise NotImplementedError


@dataclass
class _Entry:
    config_cls: Type[ModelConfig]
    describe: Callable[[ModelConfig], Any]
    model_types: tuple


_ARCHITECTURES: Dict[str, _Entry] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          describe: Callable[[ModelConfig], Any],
                          model_types: tuple = ()) -> None:
    """Register an architecture.

    ``describe(config)`` returns a ``ModelDescription`` (see ``parts/spec.py``):
    the parts of every layer, chosen layer by layer, and the order in which the
    layers run.  ``model_types`` are values of config.json's ``model_type`` that
    select this architecture when ``architectures`` is absent.
    """
    if not name:
        raise ValueError("architecture name must not be empty")
    _ARCHITECTURES[name] = _Entry(config_cls, describe, tuple(model_types))


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def _lookup(name: str) -> _Entry:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {known_architectures()}") from None


def architecture_of(raw: Dict[str, Any]) -> str:
    """Name of the architecture a raw config.json asks for."""
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return str(archs[0])
    model_type = raw.get("model_type")
    if model_type is not None:
        for name, entry in _ARCHITECTURES.items():
            if model_type in entry.model_types:
                return name
    raise ConfigError(
        "config.json names no architecture: 'architectures' is missing or empty and "
        f"model_type={model_type!r} is not registered; registered: {known_architectures()}")


def config_from_dict(raw: Dict[str, Any]) -> ModelConfig:
    entry = _lookup(architecture_of(raw))
    cfg = entry.config_cls.from_dict(raw)
    cfg.validate()
    return cfg


def load_config(model_dir) -> ModelConfig:
    """Read ``config.json`` from a model folder (or from beside a .safetensors file)."""
    path = Path(model_dir)
    if path.is_file():
        path = path.parent
    cfg_path = path / "config.json"
    if not cfg_path.is_file():
        raise ConfigError(f"no config.json in {path}")
    try:
        raw = json.loads(cfg_path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{cfg_path}: not valid JSON ({exc})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{cfg_path}: top level must be an object")
    return config_from_dict(raw)


def describe_model(config: ModelConfig):
    """The model description (layer specs and run order) of a configuration."""
    return _lookup(config.architecture).describe(config)


def require(raw: Dict[str, Any], key: str, kind=int):
    """Fetch a required config.json key with a typed error."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    return coerce(raw[key], key, kind)


def optional(raw: Dict[str, Any], key: str, default, kind=int):
    if key not in raw or raw[key] is None:
        return default
    return coerce(raw[key], key, kind)


def coerce(value, key: str, kind):
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise ConfigError(f"config.json: {key!r} must be an integer, got {value!r}")
        return int(value)
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: {key!r} must be a number, got {value!r}")
        return float(value)
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config.json: {key!r} must be true or false, got {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config.json: {key!r} must be a string, got {value!r}")
        return value
    raise TypeError(kind)
