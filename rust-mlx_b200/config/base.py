"""Typed configuration: reading config.json keys into dataclasses.

A configuration class lists the keys of its architecture's config.json as typed
fields.  Keys that the architecture does not know are ignored, as the reference
does through serde's defaults (src/dense.rs:12-25).  Every problem found in one
file is reported in one ``ConfigError``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields, MISSING
from typing import Any


class ConfigError(ValueError):
    """config.json is missing, malformed, or describes a model that cannot be built."""


@dataclass
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses add fields; ``from_dict`` fills them by name, applies ``_aliases``
    (key chains such as ``rope_parameters.rope_theta``), checks types and then
    calls ``validate`` which returns a list of problems.
    """

    model_type: str = ""
    architectures: tuple = ()

    # field name -> list of dotted key paths tried in order when the plain key is absent
    _aliases = {}
    # names of the fields that config.json has to state
    _required = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        problems = []
        values = {}
        for f in fields(cls):
            found, value = _lookup(raw, f.name, cls._aliases.get(f.name, ()))
            if not found or value is None:
                if f.name in cls._required or (f.default is MISSING and f.default_factory is MISSING):
                    problems.append(f"missing required key '{f.name}'")
                continue
            try:
                values[f.name] = _coerce(f.name, f.type, value)
            except ConfigError as e:
                problems.append(str(e))
        if problems:
            raise ConfigError("invalid configuration: " + "; ".join(problems))
        cfg = cls(**values)
        cfg._raw = dict(raw)
        problems = cfg.validate()
        if problems:
            raise ConfigError("invalid configuration: " + "; ".join(problems))
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "ModelConfig":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> list:
        return []

    def to_dict(self) -> dict:
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            if isinstance(v, tuple):
                v = list(v)
            out[f.name] = v
        return out


def read_config_json(path: str) -> dict:
    """Read ``path`` (a config.json, or a folder that holds one)."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r") as fh:
            return json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None


def _lookup(raw: dict, name: str, aliases) -> tuple:
    if name in raw and raw[name] is not None:
        return True, raw[name]
    for path in aliases:
        node: Any = raw
        ok = True
        for key in path.split("."):
            if isinstance(node, dict) and key in node and node[key] is not None:
                node = node[key]
            else:
                ok = False
                break
        if ok:
            return True, node
    return False, None


def _coerce(name: str, annotation: Any, value: Any) -> Any:
    kind = annotation if isinstance(annotation, str) else getattr(annotation, "__name__", str(annotation))
    kind = kind.replace("Optional[", "").rstrip("]")
    if kind == "int":
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise ConfigError(f"key '{name}' must be an integer, got {value!r}")
        return int(value)
    if kind == "float":
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"key '{name}' must be a number, got {value!r}")
        return float(value)
    if kind == "bool":
        if not isinstance(value, bool):
            raise ConfigError(f"key '{name}' must be true or false, got {value!r}")
        return value
    if kind == "str":
        if not isinstance(value, str):
            raise ConfigError(f"key '{name}' must be a string, got {value!r}")
        return value
    if kind == "tuple":
        if isinstance(value, (list, tuple)):
            return tuple(value)
        return (value,)
    return value
