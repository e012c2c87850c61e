"""Typed configurations and the architecture registry.  Importing registers the built-in architectures."""
from .registry import (ConfigError, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .qwen3 import Qwen3Config
from .gigopel import GigopelConfig
from .sokirax import SokiraxConfig
from .felolorn import FelolornConfig
from .dinuzen import DinuzenConfig

__all__ = ["ConfigError", "config_from_dict", "load_config", "register_architecture", "registered_architectures",
           "BlockSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule", "Qwen3Config", "GigopelConfig", "SokiraxConfig", "FelolornConfig", "DinuzenConfig"]
