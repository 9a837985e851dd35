from .llama import ConfigError, LlamaConfig, RopeScaling
from .registry import (architecture_of, config_from_dict, read_config, register_architecture,
                       registered_architectures, spec_of)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = [
    "ConfigError", "LlamaConfig", "RopeScaling", "architecture_of", "config_from_dict", "read_config",
    "register_architecture", "registered_architectures", "spec_of", "LayerSpec", "ModelSpec", "PartSpec",
]
