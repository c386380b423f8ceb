"""One registry from an architecture's name (``architectures[0]`` of
config.json) to its configuration class, whose ``model_spec`` describes the
model.  Reference: the ``ModelFamily`` seam (``src/family/mod.rs:11-82``) and
``ModelArch::from`` (``src/core/spec.rs:62-74``)."""
from __future__ import annotations

from .base import ConfigError, ModelConfig, read_config_json

_ARCHITECTURES: dict = {}


def register_architecture(name: str, config_class) -> None:
    """Make ``name`` loadable.  ``config_class`` needs ``from_dict``, ``to_dict`` and
    ``model_spec`` (see :class:`~airframe_b200.config.base.ModelConfig`)."""
    if name in _ARCHITECTURES and _ARCHITECTURES[name] is not config_class:
        raise ConfigError(f"architecture '{name}' is registered already")
    _ARCHITECTURES[name] = config_class


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_name(data: dict) -> str:
    archs = data.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: key 'architectures' must be a list that names the model class")
    return archs[0]


def config_from_dict(data: dict) -> ModelConfig:
    name = architecture_name(data)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"config.json: unknown architecture '{name}' (known: {known_architectures()})")
    return _ARCHITECTURES[name].from_dict(data)


def config_from_folder(folder) -> ModelConfig:
    return config_from_dict(read_config_json(folder))
