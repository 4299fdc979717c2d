"""Typed configurations and the registry from architecture name to configuration."""
from .registry import (ConfigError, config_class, config_from_dict, config_from_file, config_from_folder,
                       known_architectures, register_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .llama import Llama3RopeScaling, LlamaConfig

__all__ = ["ConfigError", "config_class", "config_from_dict", "config_from_file", "config_from_folder",
           "known_architectures", "register_architecture", "LayerSpec", "ModelSpec", "PartSpec",
           "ScheduleEntry", "default_schedule", "Llama3RopeScaling", "LlamaConfig"]
