"""libllm_b200: a small model library with generation of its own for one B200.

A folder with config.json and safetensors goes in, tokens come out.  See ``Model`` for
the entry point, ``engine`` for the step function and the generation loop, ``parts`` for
what layers are made of and ``config`` for the registry of architectures."""
from . import models  # noqa: F401  (registers the built-in architectures)
from .api import Chunk, Device, Model
from .config import load_config, register_architecture
from .engine import Engine, SamplingParams, StepItem, generate
from .errors import (CacheError, ConfigError, ExtensionError, InvalidArgError, LlmError, UnsupportedError,
                     WeightsError)

__version__ = "0.1.0"
__all__ = ["Chunk", "Device", "Model", "load_config", "register_architecture", "Engine", "SamplingParams",
           "StepItem", "generate", "CacheError", "ConfigError", "ExtensionError", "InvalidArgError",
           "LlmError", "UnsupportedError", "WeightsError"]
