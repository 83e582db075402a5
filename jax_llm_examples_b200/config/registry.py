"""One registry from an architecture's name to its configuration class and model builder.

``config.json["architectures"][0]`` names the architecture everywhere in the framework:
loading, random weights, the engine and trace replay all go through :func:`resolve`.
The reference has no registry (one module per model; the user imports
``llama4_jax.model``, llama4/main.py:27); a registry is what lets a second architecture be
added without touching the engine.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, Mapping

from .base import ConfigError


@dataclasses.dataclass(frozen=True)
class Architecture:
    """What an architecture must provide.

    ``parse_config(config_json) -> cfg``: typed configuration from the file's keys.
    ``tensor_specs(cfg) -> dict[name, TensorSpec]``: every tensor the model folder must hold.
    ``build(cfg, tensors, runtime) -> DecoderModel``: the model put together from parts.
    """

    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]
    tensor_specs: Callable[[Any], dict]
    build: Callable[..., Any]
    canonical_name: Callable[[str], str | None] | None = None  # file tensor name -> spec name (None = ignore)


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *aliases: str) -> None:
    for n in (arch.name, *aliases):
        _ARCHITECTURES[n] = arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def resolve(config_json: Mapping[str, Any]) -> Architecture:
    _ensure_builtin()
    archs = config_json.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config.json: key 'architectures' (a list with the model's class name) is missing")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"config.json: unknown architecture {name!r}; known: {', '.join(sorted(_ARCHITECTURES))}")
    return _ARCHITECTURES[name]


def _ensure_builtin() -> None:
    """Imports every module of the ``models`` package (each registers its architectures when imported), so an
    architecture added in-tree is one new file there.  Late: model modules import parts, which import this package."""
    import importlib
    import pkgutil

    from .. import models

    for m in pkgutil.iter_modules(models.__path__):
        importlib.import_module(f"{models.__name__}.{m.name}")
