"""One registry from an architecture's name to its configuration class and builder,
and one from a part's kind to its class.

The reference has no registry: the ``architectures`` string is only printed
(src/engine/engine_server.cpp:429-432).  Here ``config.json`` chooses the model
everywhere (engine, replay, command line) through :func:`load_config` and
:func:`model_spec_for`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Type

from .model_config import ConfigError, ModelConfig, architecture_name, read_config_json
from .model_spec import ModelSpec


@dataclass
class Architecture:
    name: str
    config_from_dict: Callable[[Dict[str, Any], str], ModelConfig]
    build_spec: Callable[[ModelConfig], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[str, Dict[str, Type]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "embedding": {}, "head": {}}


def register_architecture(name: str, config_from_dict, build_spec, replace: bool = False) -> None:
    """Make ``name`` (as written in ``architectures[0]``) loadable."""
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec)


def register_part(role: str, kind: str, cls: Type, replace: bool = False) -> None:
    """Make a part class buildable from ``PartSpec(kind=...)`` in the given role
    (``mixer``, ``ffn``, ``norm``, ``position``, ``embedding`` or ``head``)."""
    if role not in _PARTS:
        raise ValueError(f"unknown part role {role!r}; roles are {sorted(_PARTS)}")
    if kind in _PARTS[role] and not replace:
        raise ValueError(f"{role} part {kind!r} is already registered")
    _PARTS[role][kind] = cls


def part_class(role: str, kind: str) -> Type:
    _ensure_builtin()
    try:
        return _PARTS[role][kind]
    except KeyError:
        raise ConfigError(
            f"unknown {role} kind {kind!r}; registered: {sorted(_PARTS.get(role, {}))}") from None


def known_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    # Importing the packages registers what they define.
    from .. import models  # noqa: F401
    from .. import parts  # noqa: F401


def config_from_dict(raw: Dict[str, Any], where: str = "config.json") -> ModelConfig:
    _ensure_builtin()
    name = architecture_name(raw, where)
    arch = _ARCHITECTURES.get(name)
    if arch is None:
        raise ConfigError(
            f"{where}: unknown architecture {name!r}; known architectures: {known_architectures()}")
    return arch.config_from_dict(raw, where)


def load_config(model_dir: str) -> ModelConfig:
    """Read ``model_dir/config.json`` into the typed configuration of its architecture."""
    import os
    return config_from_dict(read_config_json(model_dir), os.path.join(model_dir, "config.json"))


def model_spec_for(config: ModelConfig) -> ModelSpec:
    _ensure_builtin()
    arch = _ARCHITECTURES.get(config.architecture)
    if arch is None:
        raise ConfigError(
            f"unknown architecture {config.architecture!r}; known architectures: {known_architectures()}")
    spec = arch.build_spec(config)
    spec.validate()
    return spec
