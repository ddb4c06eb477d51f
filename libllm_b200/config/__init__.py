from .base import (Architecture, ConfigReader, ModelConfig, architecture_for,
                   known_architectures, load_config, read_config_json, register_architecture)
from .llama import LlamaConfig, RopeScaling, parse_llama_config

__all__ = ["Architecture", "ConfigReader", "ModelConfig", "architecture_for", "known_architectures",
           "load_config", "read_config_json", "register_architecture", "LlamaConfig",
           "RopeScaling", "parse_llama_config"]
