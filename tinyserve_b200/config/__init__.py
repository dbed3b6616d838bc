from .model_config import (ConfigError, LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                           Qwen3Config)
from .registry import (ARCHITECTURES, architecture_of, config_from_dict, load_model_config,
                       register_architecture)
from .engine_config import EngineConfig

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec",
           "Qwen3Config", "ARCHITECTURES", "architecture_of", "config_from_dict",
           "load_model_config", "register_architecture", "EngineConfig"]
