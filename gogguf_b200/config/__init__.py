"""Typed configurations and the architecture registry.  Importing registers the built-in architectures."""
from .registry import (ConfigError, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "config_from_dict", "load_config", "register_architecture", "registered_architectures",
           "BlockSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule", "Qwen3Config"]
