"""Typed configurations and the architecture registry."""

from .base import LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry
from .registry import (architecture_name, load_config, register_architecture, resolve_config,
                       supported_architectures)
from .qwen3 import Qwen3Config

__all__ = ["LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen3Config",
           "architecture_name", "load_config", "register_architecture", "resolve_config",
           "supported_architectures"]
