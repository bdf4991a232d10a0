"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference reads config.json with a string search that returns 0 for an
absent key (src/model/model_config.cpp:13-60, 86-96), so a missing
``rms_norm_eps`` silently becomes 0.  Here every key is parsed from real JSON,
required keys raise an error that names the key, and optional keys carry the
defaults that the reference's struct declares (include/lightllm/model/model_config.h:12-30).

Nothing in this file knows a model size or an architecture: every number comes from the file, and each
architecture's own configuration class lives with its model (``models/``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional


class ConfigError(ValueError):
    """A config.json is missing a key, has a bad value, or names an unknown architecture."""


_MISSING = object()


class ConfigReader:
    """Typed access to a config dictionary with errors that name the key."""

    def __init__(self, raw: Dict[str, Any], where: str):
        self.raw = raw
        self.where = where

    def _get(self, key: str, default: Any):
        if key in self.raw and self.raw[key] is not None:
            return self.raw[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: required key '{key}' is missing")
        return default

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = 1) -> Optional[int]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {v}")
        return v

    def real(self, key: str, default: Any = _MISSING, positive: bool = True) -> float:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {v!r}")
        return v


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration: the registry key and the raw keys."""

    architecture: str
    raw: Dict[str, Any] = field(repr=False, compare=False)

    def to_json_dict(self) -> Dict[str, Any]:
        """The dictionary to write back as config.json (the architecture's own keys)."""
        return dict(self.raw)

    @property
    def eos_token_ids(self):
        """The ids that end a sequence, from ``eos_token_id`` (an integer or a list; empty when absent)."""
        v = self.raw.get("eos_token_id")
        if isinstance(v, bool) or v is None:
            return ()
        if isinstance(v, int):
            return (v,)
        if isinstance(v, (list, tuple)) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            return tuple(v)
        raise ConfigError(f"key 'eos_token_id' must be an integer or a list of integers, got {v!r}")


def architecture_name(raw: Dict[str, Any], where: str = "config.json") -> str:
    """``architectures[0]`` of a config dictionary (src/model/model_config.cpp:69-84)."""
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: required key 'architectures' must be a non-empty list of names")
    return archs[0]


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw
