"""Typed configurations, the architecture registry and the model plan."""
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, SubPart, default_schedule, prenorm_layer
from .registry import (ConfigError, config_from_dict, load_config, register_architecture,
                       registered_architectures, resolve_architecture)
from .qwen2 import Qwen2Config

__all__ = ["LayerSpec", "ModelPlan", "PartSpec", "ScheduleEntry", "SubPart", "default_schedule", "prenorm_layer", "ConfigError",
           "config_from_dict", "load_config", "register_architecture", "registered_architectures",
           "resolve_architecture", "Qwen2Config"]
