"""Typed configurations and the registry from an architecture's name to its model."""
from .registry import (ConfigError, config_class_for, config_from_dict, load_config,
                       register_architecture, registered_architectures)
from .spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry
from .llama import LlamaConfig, RopeScaling

__all__ = [
    "ArchitectureSpec", "ConfigError", "LayerSpec", "LlamaConfig", "PartSpec", "RopeScaling", "RunEntry",
    "config_class_for", "config_from_dict", "load_config", "register_architecture", "registered_architectures",
]
