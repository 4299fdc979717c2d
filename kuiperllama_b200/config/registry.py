"""One registry from an architecture's name (config.json ``architectures[0]``) to its
typed configuration class.  KuiperLLama picks the model class in ``main`` and by build
flags (demo/main.cpp:58, CMakeLists.txt:29-44); here the folder's config.json decides.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Type


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: the message names every fault."""


_ARCHITECTURES: Dict[str, type] = {}


def register_architecture(name: str) -> Callable[[type], type]:
    """Class decorator.  The class must offer ``from_dict(dict) -> config`` and the
    instance ``to_model_spec() -> ModelSpec`` and ``to_dict() -> dict``."""
    def deco(cls: type) -> type:
        if name in _ARCHITECTURES and _ARCHITECTURES[name] is not cls:
            raise ValueError(f"architecture {name!r} is already registered")
        _ARCHITECTURES[name] = cls
        return cls
    return deco


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def config_class(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; known architectures: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def config_from_dict(d: dict):
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError('config.json needs "architectures": ["<name>"]')
    return config_class(archs[0]).from_dict(d)


def config_from_folder(folder: str):
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    return config_from_file(path)


def config_from_file(path: str):
    """The typed configuration of a config.json given by its own path."""
    if not os.path.isfile(path):
        raise ConfigError(f"no such configuration file: {path!r}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return config_from_dict(d)
