"""Typed configuration: the common base and the error type.

A configuration class states, for every field, the key of the architecture's
own ``config.json`` it is read from, its type, its default and its check.
Nothing else in the framework holds a size or a constant that ``config.json``
gives; parts receive them as constructor parameters.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any


class ConfigError(ValueError):
    """A configuration key is missing, has the wrong type or an invalid value."""


def _typed(key: str, value: Any, kind: type) -> Any:
    """Convert one JSON value to ``kind`` or raise an error that names the key."""
    if kind is bool:
        if isinstance(value, bool):
            return value
        raise ConfigError(f"config key '{key}': expected true/false, got {value!r}")
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value)
            raise ConfigError(f"config key '{key}': expected an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config key '{key}': expected a number, got {value!r}")
        return float(value)
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config key '{key}': expected a string, got {value!r}")
        return value
    raise TypeError(f"unsupported field type {kind!r} for key '{key}'")


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses are frozen dataclasses whose field names are the keys of
    ``config.json``.  ``ALIASES`` maps other spellings of a key to the field;
    ``OPTIONAL_NULL`` names fields for which JSON ``null`` means "use the
    default rule" (resolved in ``__post_init__``).
    """

    architecture: str

    ALIASES = {}
    IGNORED_KEYS = ()

    @classmethod
    def from_dict(cls, raw: dict, architecture: str | None = None) -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        raw = dict(raw)
        for alias, key in cls.ALIASES.items():
            if alias in raw and key not in raw:
                raw[key] = raw[alias]
        values = {}
        for f in fields(cls):
            if f.name == "architecture":
                continue
            if f.name in raw and raw[f.name] is not None:
                kind = f.metadata.get("kind", type(f.default) if f.default is not None else int)
                values[f.name] = _typed(f.name, raw[f.name], kind)
        if architecture is None:
            architecture = architecture_name(raw)
        return cls(architecture=architecture, **values)

    def to_dict(self) -> dict:
        out = {"architectures": [self.architecture]}
        for f in fields(self):
            if f.name != "architecture":
                out[f.name] = getattr(self, f.name)
        return out


def architecture_name(raw: dict) -> str:
    """The name ``config.json`` gives its model class: ``architectures[0]``,
    or, when that list is absent, ``model_type``."""
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    model_type = raw.get("model_type")
    if isinstance(model_type, str):
        return "model_type:" + model_type
    raise ConfigError("config.json names no architecture: neither 'architectures' nor 'model_type' is set")


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            return json.load(handle)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in model folder '{model_dir}'") from None
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path} is not valid JSON: {error}") from None
