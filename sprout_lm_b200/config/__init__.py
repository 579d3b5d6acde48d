from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .registry import (architecture_name, load_config, parse_config, register_architecture,
                       registered_architectures)
from .qwen2 import Qwen2Config

register_architecture(Qwen2Config.architecture, Qwen2Config, model_types=(Qwen2Config.model_type,))

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config",
           "architecture_name", "load_config", "parse_config", "register_architecture",
           "registered_architectures"]
