from .base import BaseModelArgs, ConfigError, load_config
from .registry import (Architecture, get_architecture, get_model_classes, register_architecture,
                       registered_architectures)

__all__ = ["BaseModelArgs", "ConfigError", "load_config", "Architecture", "get_architecture",
           "get_model_classes", "register_architecture", "registered_architectures"]
