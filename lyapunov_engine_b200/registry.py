"""One registry from an architecture's name to what builds its model.

``architectures[0]`` of config.json (else ``model_type``) selects a function
that turns the raw config.json into a ``ModelSpec``.  The reference has no
registry: its command line calls the Llama loader directly
(python/lyapunov_engine/entrypoints/cli.py:20).
"""
from __future__ import annotations

from typing import Callable

from .config.base import ConfigError
from .parts.base import ModelSpec

_ARCHITECTURES: dict[str, Callable[[dict], ModelSpec]] = {}


def register_architecture(name: str, spec_builder: Callable[[dict], ModelSpec] | None = None):
    """``register_architecture("XForCausalLM", fn)`` or as a decorator."""
    def put(fn):
        _ARCHITECTURES[name] = fn
        return fn
    return put(spec_builder) if spec_builder is not None else put


def architecture_name(raw_config: dict) -> str:
    archs = raw_config.get("architectures") or []
    if archs:
        return archs[0]
    if raw_config.get("model_type"):
        return raw_config["model_type"]
    raise ConfigError("config.json names no architecture (neither 'architectures' nor 'model_type')")


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def spec_for(raw_config: dict) -> ModelSpec:
    name = architecture_name(raw_config)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered (known: {', '.join(known_architectures())})")
    return _ARCHITECTURES[name](raw_config)


def _register_builtin() -> None:
    from .models.llama import llama_spec

    register_architecture("LlamaForCausalLM", llama_spec)
    register_architecture("llama", llama_spec)


_register_builtin()
