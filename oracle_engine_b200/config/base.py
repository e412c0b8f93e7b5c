"""Typed model configuration and the one registry from architecture name to model.

A model folder's config.json names its architecture in `architectures[0]`.  The registry
maps that name to an `Architecture`: the typed configuration class that reads the
architecture's own config.json keys, and the function that turns a configuration into a
`ModelSpec` (the data description of the layers, see parts/spec.py).  Everything else
(weights, cache, step function, generation, replay, bench) is shared between
architectures.

The reference keeps its sizes in `ModelConfig` (core/model.hpp:10-27), filled from GGUF
metadata in `Model::load` (core/model.cpp:48-64), and refuses architectures it cannot run
(core/model.cpp:32-46); this module does the same from config.json.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable


class ConfigError(ValueError):
    """A config.json that cannot be used: the message names the key and the reason."""


@dataclass
class Architecture:
    name: str
    config_cls: type
    build_spec: Callable[[Any], Any]      # config -> parts.spec.ModelSpec


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable) -> None:
    if name in ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


def get_architecture(name: str) -> Architecture:
    try:
        return ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture {name!r}; registered: {known}") from None


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {folder}")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def architecture_name(raw: dict) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or len(archs) < 1 or not isinstance(archs[0], str):
        raise ConfigError("config.json: `architectures` must be a list with the model class name")
    return archs[0]


def load_config(folder):
    """config.json of `folder` -> (typed configuration, Architecture)."""
    raw = read_config_json(folder)
    arch = get_architecture(architecture_name(raw))
    return arch.config_cls.from_dict(raw), arch


class _Reader:
    """Typed access to config.json keys with errors that name the key."""

    def __init__(self, raw: dict):
        self.raw = raw

    def _get(self, key, default, required):
        if key not in self.raw or self.raw[key] is None:
            if required:
                raise ConfigError(f"config.json: missing required key `{key}`")
            return default
        return self.raw[key]

    def integer(self, key, default=None, required=True, minimum=1) -> int:
        v = self._get(key, default, required)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: `{key}` must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"config.json: `{key}` must be >= {minimum}, got {v}")
        return v

    def number(self, key, default=None, required=True, positive=True) -> float:
        v = self._get(key, default, required)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: `{key}` must be a number, got {v!r}")
        if positive and not v > 0:
            raise ConfigError(f"config.json: `{key}` must be > 0, got {v}")
        return float(v)

    def boolean(self, key, default=False) -> bool:
        v = self._get(key, default, False)
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: `{key}` must be true or false, got {v!r}")
        return v

    def id_list(self, key) -> tuple[int, ...]:
        v = self.raw.get(key)
        if v is None:
            return ()
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if isinstance(v, list) and all(isinstance(i, int) and not isinstance(i, bool) for i in v):
            return tuple(v)
        raise ConfigError(f"config.json: `{key}` must be an integer or a list of integers, got {v!r}")
