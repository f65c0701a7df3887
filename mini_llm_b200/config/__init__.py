from .base import ConfigError, ModelConfig, architecture_name, read_config_json
from .gpt2 import Gpt2Config
from .registry import (config_from_dict, config_from_folder, describe_model, known_architectures,
                       lookup_architecture, register_architecture)

__all__ = ["ConfigError", "ModelConfig", "Gpt2Config", "architecture_name", "read_config_json",
           "config_from_dict", "config_from_folder", "describe_model", "known_architectures",
           "lookup_architecture", "register_architecture"]
