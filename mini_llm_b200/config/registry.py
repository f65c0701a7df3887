"""One registry from an architecture's name to its configuration class and to
the function that describes its model.

The reference has no registry: one model is hard-wired and model names only
label its server (pytorch/src/mini_llm/batched_main.py:76-77).  Here the name
comes from ``config.json`` (``architectures[0]``, else ``model_type``) and
selects, everywhere in the framework, how the folder is read.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .base import ConfigError, ModelConfig, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    describe: Callable          # (config) -> parts.spec.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, describe: Callable, aliases=()) -> None:
    """Make ``name`` (and ``aliases``, e.g. ``"model_type:gpt2"``) known."""
    arch = Architecture(name, config_class, describe)
    for key in (name, *aliases):
        _ARCHITECTURES[key] = arch


def known_architectures() -> list[str]:
    return sorted(k for k in _ARCHITECTURES if not k.startswith("model_type:"))


def lookup_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{name}'; known: {', '.join(known_architectures())}") from None


def config_from_dict(raw: dict) -> ModelConfig:
    arch = lookup_architecture(architecture_name(raw))
    return arch.config_class.from_dict(raw, architecture=arch.name)


def config_from_folder(model_dir: str) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))


def describe_model(config: ModelConfig):
    """The model description (parts, layers, run order) of ``config``."""
    return lookup_architecture(config.architecture).describe(config)


_builtin_loaded = False


def _load_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from ..models import gpt2  # noqa: F401  (registers itself)
