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


class ConfigError(ValueError):
    pass


def register_architecture(name: str, config_class: type) -> None:
    """``config_class`` needs ``from_dict(d)``, ``to_dict()`` and ``to_model_spec()``."""
    for attr in ("from_dict", "to_dict", "to_model_spec"):
        if not hasattr(config_class, attr):
            raise TypeError(f"{config_class.__name__} lacks {attr}()")
    _ARCHITECTURES[name] = config_class


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture {name!r} is not supported; registered: {registered_architectures()}") from None


def config_from_dict(d: dict):
    """Chooses the class by ``architectures`` (first registered name wins)."""
    names = d.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    if not names:
        raise ConfigError(f"config.json names no architecture; registered: {registered_architectures()}")
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n].from_dict(d)
    raise ConfigError(f"none of {names} is supported; registered: {registered_architectures()}")


def load_config(model_dir: str):
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
    return config_from_dict(d)
