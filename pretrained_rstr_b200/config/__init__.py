from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, RunEntry, replace
from .gpt2 import GPT2Config
from .registry import (Architecture, dispatch_keys, lookup, read_config,
                       register_architecture, registered)

__all__ = ["ConfigError", "LayerSpec", "ModelConfig", "PartSpec", "RunEntry", "replace",
           "GPT2Config", "Architecture", "dispatch_keys", "lookup", "read_config",
           "register_architecture", "registered"]
