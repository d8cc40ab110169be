"""One registry from an architecture's name to its configuration reader and model
description (reference src/runtime/model_registry.cpp:74-113: ``model_type`` -> parse +
create_runner, unknown types are refused by name)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Sequence, Tuple

from .base import ConfigError, load_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]
    model_spec: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable[[Dict[str, Any]], Any],
                          model_spec: Callable[[Any], Any], aliases: Sequence[str] = ()) -> None:
    arch = Architecture(name, parse_config, model_spec)
    for key in (name, *aliases):
        _ARCHITECTURES[key] = arch


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted({a.name for a in _ARCHITECTURES.values()}))


def resolve_architecture(config: Dict[str, Any]) -> Architecture:
    """By ``model_type``, else by the first known entry of ``architectures``."""
    mt = config.get("model_type")
    if isinstance(mt, str) and mt in _ARCHITECTURES:
        return _ARCHITECTURES[mt]
    for name in config.get("architectures") or []:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    if mt is None:
        raise ConfigError("config field 'model_type': missing")
    raise ConfigError(f"unsupported model_type: {mt} (known: {', '.join(registered_architectures())})")


def open_model_dir(model_dir: str):
    """(architecture, typed config) of the model folder."""
    data = load_config_json(model_dir)
    arch = resolve_architecture(data)
    return arch, arch.parse_config(data)
