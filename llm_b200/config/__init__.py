from .base import ConfigReader, read_config_json
from .llama import LlamaConfig
from .registry import (config_class_for, config_from_dict, known_architectures, load_config,
                       register_architecture)

register_architecture(LlamaConfig.architecture, LlamaConfig)

__all__ = ["ConfigReader", "read_config_json", "LlamaConfig", "config_class_for",
           "config_from_dict", "known_architectures", "load_config", "register_architecture"]
