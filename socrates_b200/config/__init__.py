from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .qwen3 import ConfigError, Qwen3Config
from .registry import (config_from_dict, known_architectures, load_config,
                       register_architecture, unregister_architecture)
from .engine import EngineConfig

__all__ = [
    "LayerSpec", "ModelPlan", "PartSpec", "RunEntry", "ConfigError", "Qwen3Config",
    "config_from_dict", "known_architectures", "load_config", "register_architecture",
    "unregister_architecture", "EngineConfig",
]
