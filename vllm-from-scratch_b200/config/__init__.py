"""Configuration: the model's own config.json as a typed object, the engine's
knobs, and the registry from an architecture's name to what builds it."""

from .engine_config import (CacheConfig, EngineConfig, ModelConfig, SchedulerConfig,
                            VllmConfig, canonical_dtype)
from .bemuzen_config import BemuzenConfig
from .lobuzen_config import LobuzenConfig
from .mupuvik_config import MupuvikConfig
from .nodopel_config import NodopelConfig
from .model_config import ConfigError, Qwen3Config
from .registry import (ArchitectureEntry, get_architecture, load_model_config,
                       register_architecture, registered_architectures)

__all__ = [
    "ArchitectureEntry", "BemuzenConfig", "CacheConfig", "ConfigError", "EngineConfig", "LobuzenConfig", "ModelConfig", "MupuvikConfig", "NodopelConfig",
    "Qwen3Config", "SchedulerConfig", "VllmConfig", "canonical_dtype", "get_architecture",
    "load_model_config", "register_architecture", "registered_architectures",
]
