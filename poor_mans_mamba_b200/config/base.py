"""Reading ``config.json`` and the small vocabulary shared by all architecture configs.

The reference reads every key as required and reports the key's name on failure
(include/io/utils.h:12-18); its loader first replaces the non-JSON tokens that
Hugging Face writers emit (src/io/utils.cpp:19-42).  Both behaviours are kept; keys
that only tune an optional feature may fall back to a neutral default, sizes may not.
"""
from __future__ import annotations

import json
import os
import re
from typing import Any, Callable, Dict, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the named architecture."""


_MISSING = object()


def load_config_json(model_dir: str) -> Dict[str, Any]:
    """Parse ``<model_dir>/config.json``.  ``Infinity``/``-Infinity``/``NaN`` outside
    strings are mapped to 1e308 / -1e308 / null before parsing, as the reference does."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            text = fh.read()
    except OSError as exc:
        raise ConfigError(f"cannot read {path}: {exc}") from exc
    text = re.sub(r"(?<![\w\"])-Infinity(?![\w\"])", "-1e308", text)
    text = re.sub(r"(?<![\w\"])Infinity(?![\w\"])", "1e308", text)
    text = re.sub(r"(?<![\w\"])NaN(?![\w\"])", "null", text)
    try:
        data = json.loads(text)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return data


class KeyReader:
    """Typed access to a config dict with the key's name in every error."""

    def __init__(self, data: Dict[str, Any]):
        self.data = data

    def _get(self, key: str, default: Any) -> Any:
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            raise ConfigError(f"config field '{key}': missing")
        return default

    def _typed(self, key: str, default: Any, check: Callable[[Any], bool], conv: Callable[[Any], Any],
               what: str) -> Any:
        val = self._get(key, default)
        if val is default and default is not _MISSING:
            return default
        if not check(val):
            raise ConfigError(f"config field '{key}': expected {what}, got {val!r}")
        return conv(val)

    def int(self, key: str, default: Any = _MISSING) -> int:
        return self._typed(key, default, lambda v: isinstance(v, int) and not isinstance(v, bool), int,
                           "an integer")

    def float(self, key: str, default: Any = _MISSING) -> float:
        return self._typed(key, default,
                           lambda v: isinstance(v, (int, float)) and not isinstance(v, bool), float,
                           "a number")

    def bool(self, key: str, default: Any = _MISSING) -> bool:
        return self._typed(key, default, lambda v: isinstance(v, bool), bool, "true or false")

    def str(self, key: str, default: Any = _MISSING) -> str:
        return self._typed(key, default, lambda v: isinstance(v, str), str, "a string")

    def float_list(self, key: str, length: int, default: Any = _MISSING):
        val = self._get(key, default)
        if val is default and default is not _MISSING:
            return tuple(default)
        ok = isinstance(val, (list, tuple)) and all(
            isinstance(v, (int, float)) and not isinstance(v, bool) for v in val)
        if not ok:
            raise ConfigError(f"config field '{key}': expected a list of numbers, got {val!r}")
        if len(val) != length:
            raise ConfigError(f"config field '{key}': must have length {length}, got {len(val)}")
        return tuple(float(v) for v in val)

    def optional_int(self, key: str) -> Optional[int]:
        if key not in self.data or self.data[key] is None:
            return None
        return self.int(key)
