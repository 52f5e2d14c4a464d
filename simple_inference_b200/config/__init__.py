from .model_config import ConfigError, LlamaConfig, ModelConfig, RopeScaling
from .registry import (Architecture, architecture_of, known_architectures, read_config,
                       register_architecture)

__all__ = ["ConfigError", "LlamaConfig", "ModelConfig", "RopeScaling", "Architecture",
           "architecture_of", "known_architectures", "read_config", "register_architecture"]
