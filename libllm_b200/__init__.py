"""libllm_b200: a small model library with generation of its own for one B200.

A folder with config.json and safetensors goes in, tokens come out.  The library itself is
C++ and CUDA (the host library ``libllm_b200`` with the C interface of ``include/llm.h``, and
the kernel families of ``csrc``); this package is its Python face: ``Model`` for the entry
point, ``engine`` for the step function and the generation loop, ``parts`` for registering parts
of one's own and ``config`` for the registry of architectures."""
from .api import Chunk, Device, Model
from .config import load_config, register_architecture
from .engine import Engine, SamplingParams, StepItem, generate
from .errors import (CacheError, ConfigError, ExtensionError, InvalidArgError, LlmError, UnsupportedError,
                     WeightsError)

__version__ = "0.2.0"
__all__ = ["Chunk", "Device", "Model", "load_config", "register_architecture", "Engine", "SamplingParams",
           "StepItem", "generate", "CacheError", "ConfigError", "ExtensionError", "InvalidArgError",
           "LlmError", "UnsupportedError", "WeightsError"]
