from .registry import (Architecture, ConfigError, architecture_of, known_architectures, load_config,
                       read_config_json, register_architecture)
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .llama import LlamaConfig, RopeScaling

__all__ = ["Architecture", "ConfigError", "architecture_of", "known_architectures", "load_config",
           "read_config_json", "register_architecture", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec",
           "LlamaConfig", "RopeScaling"]
