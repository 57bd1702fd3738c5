"""Configuration: typed per-architecture classes, the neutral ``ModelSpec``
they produce, and the registry that finds the class for a ``config.json``."""
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (architecture_name, config_from_dict, config_from_dir,
                       known_architectures, register_architecture)
from .qwen3 import Qwen3Config

register_architecture("Qwen3ForCausalLM", Qwen3Config, model_type="qwen3")

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
           "architecture_name", "config_from_dict", "config_from_dir",
           "known_architectures", "register_architecture"]
