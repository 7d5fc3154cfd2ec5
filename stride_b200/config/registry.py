"""One registry from an architecture's name (``architectures`` in config.json) to
its typed configuration class. The class reads the architecture's own keys and
turns itself into a ``ModelSpec``; the engine builds every model from that.

The reference keeps a set of supported names and one model class
(python/stride_worker/model.py:36-40,193-199); an unknown name is an error that
lists what is registered.
"""

from __future__ import annotations

import json
import os

_ARCHITECTURES: dict[str, type] = {}
_MODEL_TYPES: dict[str, str] = {}       # config.json's `model_type` -> architecture name


class ConfigError(ValueError):
    pass


def register_architecture(name: str, config_class: type, model_type: str | None = None) -> None:
    """``config_class`` needs ``from_dict(d)``, ``to_dict()`` and ``to_model_spec()``. It may also have
    ``complete_from_checkpoint(d, tensor_names) -> dict``: keys that config.json leaves out and that the
    checkpoint's contents settle. ``model_type`` names the architecture for a config.json that gives no
    ``architectures``."""
    for attr in ("from_dict", "to_dict", "to_model_spec"):
        if not hasattr(config_class, attr):
            raise TypeError(f"{config_class.__name__} lacks {attr}()")
    _ARCHITECTURES[name] = config_class
    if model_type is not None:
        _MODEL_TYPES[model_type] = name


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture {name!r} is not supported; registered: {registered_architectures()}") from None


def config_class_of(d: dict) -> type:
    """Chooses the class by ``architectures`` (first registered name wins); a config.json that names none is
    placed by its ``model_type``."""
    names = d.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    if not names and d.get("model_type") in _MODEL_TYPES:
        names = [_MODEL_TYPES[d["model_type"]]]
    if not names:
        raise ConfigError(f"config.json names no architecture; registered: {registered_architectures()}")
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    raise ConfigError(f"none of {names} is supported; registered: {registered_architectures()}")


def config_from_dict(d: dict, tensor_names=None):
    """The typed configuration of ``d``. With ``tensor_names`` (what the checkpoint holds) the class may first
    settle keys that config.json leaves out."""
    cls = config_class_of(d)
    if tensor_names is not None and hasattr(cls, "complete_from_checkpoint"):
        d = cls.complete_from_checkpoint(dict(d), set(tensor_names))
    return cls.from_dict(d)


def load_config(model_dir: str, tensor_names=None):
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json under {model_dir}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config_from_dict(d, tensor_names)
