"""Typed configurations and the architecture registry."""
from .base import (ConfigError, KeyReader, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                   ScheduleEntry, read_config_json)
from .gemma2 import Gemma2Config
from .registry import (architecture_name, config_from_dict, config_from_folder,
                       known_architectures, register_architecture)

register_architecture(Gemma2Config.architecture, Gemma2Config)

__all__ = [
    "ConfigError", "KeyReader", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "ScheduleEntry",
    "read_config_json", "Gemma2Config", "architecture_name", "config_from_dict",
    "config_from_folder", "known_architectures", "register_architecture",
]
