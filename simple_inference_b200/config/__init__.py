from .model_config import ConfigError, LlamaConfig, ModelConfig, RopeScaling
from .sapanex_config import SapanexConfig
from .registry import (Architecture, architecture_of, known_architectures, read_config,
                       register_architecture)

__all__ = ["ConfigError", "LlamaConfig", "ModelConfig", "RopeScaling", "SapanexConfig", "Architecture",
           "architecture_of", "known_architectures", "read_config", "register_architecture"]
