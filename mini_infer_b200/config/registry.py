"""Architecture registry: ``config.json``'s ``architectures[0]`` -> how to build it.

An architecture is registered as a pair of callables:

``parse(raw: dict) -> config``
    turns the raw ``config.json`` mapping into a typed, validated configuration;
``assemble(config) -> ModelSpec``
    turns that configuration into a description of parts (``parts.spec``):
    which mixer, feed-forward, norm and position encoding every layer has, in
    which order layers run, and under which tensor names their weights live.

Nothing else in the package knows an architecture by name.  The reference keeps
the same contract in ``models/__init__.py:24-70`` (a dict keyed by the HF
architecture string, unknown names raise a ``ValueError`` listing the known
ones, an empty ``architectures`` list raises too).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that cannot be turned into a model."""


@dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable[[Mapping[str, Any]], Any]
    assemble: Callable[[Any], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    parse: Callable[[Mapping[str, Any]], Any],
    assemble: Callable[[Any], Any],
    *,
    replace: bool = False,
) -> Architecture:
    """Register ``name`` (the string found in ``architectures[0]``)."""
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    arch = Architecture(name=name, parse=parse, assemble=assemble)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {sorted(_ARCHITECTURES)}"
        ) from None


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    archs = raw.get("architectures")
    if not archs:
        raise ConfigError("config.json has no 'architectures' entry")
    if not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError(f"'architectures' must be a list of names, got {archs!r}")
    return lookup_architecture(archs[0])


def read_config_json(model_dir: str | os.PathLike) -> dict[str, Any]:
    path = os.path.join(os.fspath(model_dir), "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {os.fspath(model_dir)!r}")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def load_config(model_dir_or_raw: str | os.PathLike | Mapping[str, Any]):
    """``(architecture, typed config)`` from a model folder or a raw mapping."""
    if isinstance(model_dir_or_raw, Mapping):
        raw = dict(model_dir_or_raw)
    else:
        raw = read_config_json(model_dir_or_raw)
    arch = architecture_of(raw)
    return arch, arch.parse(raw)


_builtin_loaded = False


def _load_builtin() -> None:
    """Import the architecture files that ship with the package (once)."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    from ..models import llama  # noqa: F401  (registers itself on import)
