"""One registry from an architecture's name to its configuration class and model.

config.json's ``architectures[0]`` (for instance "Qwen3ForCausalLM") or, when it is
absent, ``model_type`` picks the entry.  The reference has no registry: its dense
model compares ``model_type`` with "qwen3" (src/dense.rs:316) and the binary picks
the model type.  An entry's ``build`` turns a typed configuration into a
``ModelSpec``: parts with their sizes and the schedule, no tensors yet.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .config.base import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build: Callable
    model_types: tuple = ()


_ARCHITECTURES: dict = {}


def register_architecture(name: str, config_class: type, build: Callable, model_types: tuple = ()) -> None:
    """Add (or replace) an architecture.  ``build(config) -> ModelSpec``."""
    _ARCHITECTURES[name] = Architecture(name, config_class, build, tuple(model_types))


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def find_architecture(raw: dict) -> Architecture:
    """The entry that a config.json (as a dict) names."""
    _load_builtin()
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = raw.get("model_type")
    if not names and mt is not None:
        for a in _ARCHITECTURES.values():
            if mt in a.model_types:
                return a
    asked = names[0] if names else mt
    raise ConfigError(f"unknown architecture {asked!r}; known: {', '.join(sorted(_ARCHITECTURES))}")


def load_config(path: str) -> ModelConfig:
    """Read a folder's config.json into the typed configuration of its architecture."""
    raw = read_config_json(path)
    return find_architecture(raw).config_class.from_dict(raw)


def build_model_spec(config: ModelConfig):
    raw = {"architectures": list(config.architectures), "model_type": config.model_type}
    return find_architecture(raw).build(config)


_loaded = False


def _load_builtin() -> None:
    global _loaded
    if not _loaded:
        _loaded = True
        from .models import qwen3  # noqa: F401  (registers itself)
