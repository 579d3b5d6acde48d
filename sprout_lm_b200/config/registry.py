"""One registry from an architecture's name to its configuration class.

A configuration class has ``from_dict(raw) -> config`` (raising ConfigError),
``to_dict()``, ``model_spec() -> ModelSpec`` and ``with_eos(ids)``.  The
architecture of a model folder is ``architectures[0]`` of its config.json when
that is present, otherwise its ``model_type`` (the reference's fixture has
``"architectures": null`` and is recognised by ``model_type`` alone,
src/qwen.ts:17).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

from .specs import ConfigError

_BY_ARCHITECTURE: dict[str, type] = {}
_BY_MODEL_TYPE: dict[str, str] = {}


def register_architecture(name: str, config_class: type, model_types: tuple[str, ...] = ()) -> None:
    """Make ``name`` (a config.json ``architectures`` entry) known; ``model_types`` are the
    ``model_type`` values that select it when ``architectures`` is absent."""
    _BY_ARCHITECTURE[name] = config_class
    for model_type in model_types:
        _BY_MODEL_TYPE[model_type] = name


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted(_BY_ARCHITECTURE))


def architecture_name(raw: Mapping[str, Any]) -> str:
    if not isinstance(raw, Mapping):
        raise ConfigError("config.json must hold a JSON object.")
    names = raw.get("architectures")
    if isinstance(names, list) and names:
        name = names[0]
        if name not in _BY_ARCHITECTURE:
            raise ConfigError(f"Unknown architecture {name!r}; registered: {', '.join(registered_architectures())}.")
        return name
    model_type = raw.get("model_type")
    if model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    raise ConfigError(f"Unknown model_type {model_type!r}; registered: {', '.join(sorted(_BY_MODEL_TYPE))}.")


def parse_config(raw: Mapping[str, Any]):
    """Typed configuration of the architecture that ``raw`` names."""
    return _BY_ARCHITECTURE[architecture_name(raw)].from_dict(raw)


def load_config(directory):
    """Configuration of a model folder; generation_config.json's eos_token_id, when the file
    exists, replaces config.json's (src/qwen.ts:124-128)."""
    directory = Path(directory)
    path = directory / "config.json"
    if not path.exists():
        raise ConfigError(f"{path} does not exist.")
    config = parse_config(json.loads(path.read_text()))
    generation = directory / "generation_config.json"
    if generation.exists():
        eos = json.loads(generation.read_text()).get("eos_token_id")
        if eos is not None:
            config = config.with_eos(eos)
    return config
