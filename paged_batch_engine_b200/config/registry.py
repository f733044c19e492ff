"""One registry from an architecture's name (``architectures[0]`` of config.json) to its
typed configuration and its model builder.

The reference chooses its single architecture at compile time (``-DQWEN2_SUPPORT``,
CMakeLists.txt:19-23; class picked by the demo, demo/main_qwen.cpp:60).  Here the choice
is made from ``config.json`` everywhere: loader, engine, command line and trace replay.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .specs import ConfigError


@dataclass
class Architecture:
    name: str
    config_class: Any                 # has from_dict(dict) and model_spec()
    builder: Optional[Callable] = None  # (spec, dtype, device) -> model; None: the generic decoder


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class, builder: Optional[Callable] = None,
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, builder)


def known_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def architecture_name_of(config_dict: Dict[str, Any]) -> str:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json has no 'architectures' list")
    return str(archs[0])


def load_config(path_or_dict):
    """config.json (a folder, a file or a dict) -> (Architecture, typed config)."""
    if isinstance(path_or_dict, dict):
        d = path_or_dict
    else:
        path = path_or_dict
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if not os.path.exists(path) or os.path.isdir(path):
            raise ConfigError(f"no config.json at {path}")
        with open(path, "r", encoding="utf-8") as f:
            try:
                d = json.load(f)
            except json.JSONDecodeError as e:
                raise ConfigError(f"{path} is not valid JSON: {e}") from e
    arch = get_architecture(architecture_name_of(d))
    return arch, arch.config_class.from_dict(d)
