"""Typed configurations and the architecture registry."""
from .base import ConfigError, ModelConfig
from .bomipel import BomipelConfig
from .engine import EngineConfig
from .kanavik import KanavikConfig
from .qwen2 import Qwen2Config
from .rekodra import RekodraConfig
from .registry import (
    config_class_for,
    config_from_dict,
    known_architectures,
    load_config,
    register_architecture,
)
from .tepavik import TepavikConfig
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

register_architecture(Qwen2Config)
register_architecture(TepavikConfig)
register_architecture(BomipelConfig)
register_architecture(KanavikConfig)
register_architecture(RekodraConfig)

__all__ = [
    "BomipelConfig",
    "ConfigError",
    "EngineConfig",
    "KanavikConfig",
    "LayerSpec",
    "ModelConfig",
    "ModelSpec",
    "PartSpec",
    "Qwen2Config",
    "RekodraConfig",
    "ScheduleEntry",
    "TensorSpec",
    "TepavikConfig",
    "config_class_for",
    "config_from_dict",
    "known_architectures",
    "load_config",
    "register_architecture",
]
