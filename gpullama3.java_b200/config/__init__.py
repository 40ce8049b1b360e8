"""Typed configurations and the architecture registry."""
from .base import (ConfigError, LayerSpec, ModelConfig, PartSpec, ScheduleEntry, default_schedule,
                   read_config_json)
from .registry import (Architecture, architecture_of, config_from_dict, load_config, register_architecture,
                       registered_architectures, unregister_architecture)
from .llama import LlamaConfig, RopeScaling

__all__ = ["ConfigError", "LayerSpec", "ModelConfig", "PartSpec", "ScheduleEntry", "default_schedule",
           "read_config_json", "Architecture", "architecture_of", "config_from_dict", "load_config",
           "register_architecture", "registered_architectures", "unregister_architecture", "LlamaConfig",
           "RopeScaling"]
