from .base import (Architecture, ConfigError, ModelConfig, architecture_of, load_config,
                   register_architecture, registered_architectures)
from .gemma2 import Gemma2Config

__all__ = ["Architecture", "ConfigError", "ModelConfig", "Gemma2Config", "architecture_of",
           "load_config", "register_architecture", "registered_architectures"]
