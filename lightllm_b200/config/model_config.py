"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference reads config.json with a string search that returns 0 for an
absent key (src/model/model_config.cpp:13-60, 86-96), so a missing
``rms_norm_eps`` silently becomes 0.  Here every key is parsed from real JSON,
required keys raise an error that names the key, and optional keys carry the
defaults that the reference's struct declares (include/lightllm/model/model_config.h:12-30).

Nothing in this file knows a model size: every number comes from the file.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional


class ConfigError(ValueError):
    """A config.json is missing a key, has a bad value, or names an unknown architecture."""


_MISSING = object()


class _Reader:
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


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """Configuration of ``Qwen2ForCausalLM`` (dense decoder: GQA attention with QKV bias,
    NeoX rotary positions, RMSNorm, SwiGLU, optionally tied embeddings).

    Keys and fallbacks follow src/model/model_config.cpp:86-102 (``num_key_value_heads``
    defaults to ``num_attention_heads``, head size defaults to hidden/heads); the
    defaults of ``rms_norm_eps`` and ``rope_theta`` are the struct's
    (include/lightllm/model/model_config.h:20,23).  ``head_dim``, the window keys and
    ``tie_word_embeddings`` are honoured although the reference ignores them.
    """

    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"

    @staticmethod
    def from_dict(raw: Dict[str, Any], where: str = "config.json") -> "Qwen2Config":
        r = _Reader(raw, where)
        arch = architecture_name(raw, where)
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads", heads)
        head_dim = r.integer("head_dim", None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"{where}: 'hidden_size' {hidden} is not a multiple of 'num_attention_heads' {heads} "
                    "and no 'head_dim' is given")
            head_dim = hidden // heads
        if heads % kv_heads != 0:
            raise ConfigError(
                f"{where}: 'num_attention_heads' {heads} is not a multiple of 'num_key_value_heads' {kv_heads}")
        if head_dim % 2 != 0:
            raise ConfigError(f"{where}: 'head_dim' {head_dim} must be even for rotary positions")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{where}: 'hidden_act' must be 'silu' for {arch}, got {act!r}")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"{where}: 'rope_scaling' is not supported for {arch}: {raw['rope_scaling']!r}")
        layers = r.integer("num_hidden_layers")
        use_window = r.boolean("use_sliding_window", False)
        window = r.integer("sliding_window", None)
        max_window_layers = r.integer("max_window_layers", layers, minimum=0)
        if use_window and window is None:
            raise ConfigError(f"{where}: 'use_sliding_window' is true but 'sliding_window' is missing")
        return Qwen2Config(
            architecture=arch,
            raw=dict(raw),
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=r.real("rms_norm_eps", 1e-6),
            rope_theta=r.real("rope_theta", 10000.0),
            max_position_embeddings=r.integer("max_position_embeddings"),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=max_window_layers,
            hidden_act=act,
        )

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of a layer's attention: the first ``max_window_layers`` layers see every
        earlier token; later ones see the last ``sliding_window`` tokens (self included)
        when ``use_sliding_window`` is set."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None


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
