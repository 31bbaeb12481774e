"""Typed reading of config.json.

A configuration class names every key it reads.  A key that gives a size or a
constant of the model has no default in code: when config.json lacks it the
error names the key.  Options with a default defined by the checkpoint format
itself (``tie_word_embeddings`` false, ``num_key_value_heads`` equal to the
number of heads, ``head_dim`` the quotient of width and heads) are derived, not
assumed.

The reference reads config.json with a default for every key
(python/lyapunov_engine/models/weight_loader.py:10-38) so that a folder without
a key silently becomes Llama-3.2-1B; here that is an error.
"""
from __future__ import annotations

import json
import os
from typing import Any


class ConfigError(ValueError):
    """config.json lacks a key, or holds a value the engine cannot run."""


_MISSING = object()


class KeyReader:
    """Reads keys of one config.json and remembers which were read."""

    def __init__(self, raw: dict, source: str = "config.json"):
        self.raw = raw
        self.source = source
        self.seen: set[str] = set()

    def _get(self, key: str, default=_MISSING):
        self.seen.add(key)
        value = self.raw.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                raise ConfigError(f"{self.source}: required key {key!r} is missing")
            return default
        return value

    def integer(self, key: str, default=_MISSING, minimum: int | None = 1) -> int:
        value = self._get(key, default)
        if value is None:
            return value
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"{self.source}: {key!r} must be an integer, got {value!r}")
        if minimum is not None and value < minimum:
            raise ConfigError(f"{self.source}: {key!r} must be >= {minimum}, got {value}")
        return value

    def number(self, key: str, default=_MISSING, positive: bool = True) -> float:
        value = self._get(key, default)
        if value is None:
            return value
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{self.source}: {key!r} must be a number, got {value!r}")
        if positive and not value > 0:
            raise ConfigError(f"{self.source}: {key!r} must be > 0, got {value}")
        return float(value)

    def boolean(self, key: str, default=_MISSING) -> bool:
        value = self._get(key, default)
        if not isinstance(value, bool):
            raise ConfigError(f"{self.source}: {key!r} must be true or false, got {value!r}")
        return value

    def string(self, key: str, default=_MISSING) -> str:
        value = self._get(key, default)
        if value is not None and not isinstance(value, str):
            raise ConfigError(f"{self.source}: {key!r} must be a string, got {value!r}")
        return value

    def mapping(self, key: str, default=_MISSING) -> dict | None:
        value = self._get(key, default)
        if value is not None and not isinstance(value, dict):
            raise ConfigError(f"{self.source}: {key!r} must be an object, got {value!r}")
        return value

    def id_list(self, key: str, default=_MISSING) -> tuple[int, ...]:
        """A token id or a list of them (``eos_token_id`` may be either)."""
        value = self._get(key, default)
        if value is None:
            return ()
        if isinstance(value, int) and not isinstance(value, bool):
            return (value,)
        if isinstance(value, (list, tuple)) and all(
                isinstance(v, int) and not isinstance(v, bool) for v in value):
            return tuple(value)
        raise ConfigError(f"{self.source}: {key!r} must be an id or a list of ids, got {value!r}")


def read_config_json(folder: str) -> dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: must hold a JSON object")
    return raw
