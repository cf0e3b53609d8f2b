from .base import (Architecture, ConfigError, ModelConfig, config_from_dict, load_config,
                   register_architecture, registered_architectures, resolve_architecture)
from .llama import LlamaConfig, RopeScaling

__all__ = ["Architecture", "ConfigError", "ModelConfig", "config_from_dict", "load_config",
           "register_architecture", "registered_architectures", "resolve_architecture",
           "LlamaConfig", "RopeScaling"]
