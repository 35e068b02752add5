"""The one registry from an architecture's name to its configuration class and its model description."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from ..errors import LoadError, UnsupportedError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict], Any]      # config.json (dict) -> typed configuration
    build_spec: Callable[[Any], ModelSpec]   # typed configuration -> ModelSpec
    model_types: tuple[str, ...] = ()        # config.json "model_type" values that also select it


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_json: dict) -> Architecture:
    """Chooses by `architectures[0]`, else by `model_type` (the only key the reference reads,
    src/model/config.cpp:39-42)."""
    names = config_json.get("architectures") or []
    if names:
        if names[0] in _ARCHITECTURES:
            return _ARCHITECTURES[names[0]]
        raise UnsupportedError(f"architecture '{names[0]}' is not supported (supported: {', '.join(architectures())})")
    model_type = config_json.get("model_type")
    if model_type is None:
        raise LoadError("config.json has no 'model_type'")
    for arch in _ARCHITECTURES.values():
        if model_type in arch.model_types:
            return arch
    raise UnsupportedError(f"architecture '{model_type}' is not supported (supported: "
                           f"{', '.join(sorted(t for a in _ARCHITECTURES.values() for t in a.model_types))})")


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    try:
        text = path.read_text()
    except OSError as e:
        raise LoadError(f"{path}: cannot open ({e.strerror})") from None
    try:
        cfg = json.loads(text)
    except json.JSONDecodeError as e:
        raise LoadError(f"{path}: invalid JSON: {e}") from None
    if not isinstance(cfg, dict):
        raise LoadError(f"{path}: expected a JSON object")
    return cfg


def load_config(model_dir):
    """config.json of a folder -> (architecture, typed configuration, model description)."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    cfg = arch.parse_config(raw)
    spec = arch.build_spec(cfg)
    spec.validate()
    return arch, cfg, spec
