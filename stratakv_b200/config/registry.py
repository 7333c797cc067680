"""One registry from an architecture's name (``config.json: architectures[0]``)
to its configuration class and its model description.

The reference has a single hard-wired model (``src/generation/generator.cpp:
374-511``); here the name decides, everywhere a model folder is opened.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict

from .llama import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                    # has from_dict(raw) and to_dict()
    build_spec: Callable[[Any], Any]     # config -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class, build_spec) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{name}'; known: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def read_config_json(model_dir) -> dict:
    path = Path(model_dir)
    if path.is_dir():
        path = path / "config.json"
    try:
        raw = json.loads(path.read_text())
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path}: not valid JSON ({error})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def load_config(model_dir):
    """Read ``config.json`` and return ``(architecture, typed config)``."""
    raw = read_config_json(model_dir)
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    arch = resolve_architecture(archs[0])
    return arch, arch.config_class.from_dict(raw)
