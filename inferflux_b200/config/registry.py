"""One registry from an architecture's name to its configuration class.

The reference resolves `model_type` (else `architectures[0]`) to a forward class by
string compare and answers "Unsupported model_type" otherwise
(runtime/backends/cuda/native/model_forward_factory.cpp:25-60).  Here the name maps
to a configuration class whose `to_plan()` describes the model in parts; nothing
else in the engine depends on the name.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict, Type

_ARCHITECTURES: Dict[str, type] = {}


class ConfigError(ValueError):
    """A config.json that is missing a key, has a wrong value, or names an
    architecture that is not registered."""


def register_architecture(*names: str) -> Callable[[type], type]:
    """Class decorator: `names` are the strings config.json may carry in
    `architectures[0]` or `model_type`."""
    def deco(cls: type) -> type:
        for n in names:
            _ARCHITECTURES[n] = cls
        return cls
    return deco


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: dict) -> type:
    names = []
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        names.append(str(archs[0]))
    if raw.get("model_type"):
        names.append(str(raw["model_type"]))
    if not names:
        raise ConfigError("config.json has neither `architectures` nor `model_type`")
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    for n in names:                                   # the reference lower-cases model_type
        if n.lower() in _ARCHITECTURES:
            return _ARCHITECTURES[n.lower()]
    raise ConfigError(f"unsupported architecture {names}; registered: {registered_architectures()}")


def config_from_dict(raw: dict):
    cls = resolve_architecture(raw)
    return cls.from_dict(raw)


def load_config(model_dir):
    """Typed configuration of a model folder, chosen by its config.json."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} not found: a model folder holds config.json and model.safetensors")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return config_from_dict(raw)
