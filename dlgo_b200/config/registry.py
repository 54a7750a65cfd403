"""Registry from an architecture's name to its configuration class.

The reference keeps ``archRegistry`` (models/llm/arch.go:17-64) and hands an
unknown name a default descriptor.  Here an unknown name is an error that lists
what is registered: a silent default would run the wrong formulas.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping, Protocol

from .spec import ArchitectureSpec


class ArchitectureConfig(Protocol):
    """What a registered configuration class must offer."""

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ArchitectureConfig": ...

    def to_dict(self) -> Dict[str, Any]: ...

    def architecture_spec(self) -> ArchitectureSpec: ...


_ARCHITECTURES: Dict[str, Callable[[Mapping[str, Any]], ArchitectureConfig]] = {}


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


def register_architecture(name: str, config_class: Any, *, replace: bool = False) -> None:
    """Register ``config_class`` (with ``from_dict`` / ``architecture_spec``) under ``name``."""
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = config_class


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> Any:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(registered_architectures()) or '(none)'}"
        ) from None


def config_from_dict(d: Mapping[str, Any]) -> ArchitectureConfig:
    archs = d.get("architectures")
    if isinstance(archs, str):
        archs = [archs]
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError('config.json has no "architectures" entry')
    cls = config_class_for(str(archs[0]))
    return cls.from_dict(d)


def load_config(model_dir: str) -> ArchitectureConfig:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir!r}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)
