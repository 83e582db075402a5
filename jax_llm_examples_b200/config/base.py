"""Typed configuration plumbing shared by every architecture.

A model folder's ``config.json`` is the only source of sizes and constants.  The
helpers here read keys with a declared type and raise :class:`ConfigError` naming
the key when one is missing or has the wrong type, so that no default silently
stands in for a value the file should have given.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Callable, Mapping


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration."""


_MISSING = object()


def read_key(d: Mapping[str, Any], key: str, typ: type | tuple[type, ...], default: Any = _MISSING) -> Any:
    """Return ``d[key]`` checked against ``typ``; ``default`` stands in only if given."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if typ is int and isinstance(v, bool):
        raise ConfigError(f"config.json: key '{key}' must be an integer, found a bool")
    if typ is int and isinstance(v, float) and float(v).is_integer():
        v = int(v)
    if not isinstance(v, typ):
        raise ConfigError(f"config.json: key '{key}' must be {typ}, found {type(v).__name__} ({v!r})")
    return v


def require(cond: bool, message: str) -> None:
    if not cond:
        raise ConfigError("config.json: " + message)


def load_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in model folder {model_dir}")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e


ConfigFactory = Callable[[Mapping[str, Any]], Any]
