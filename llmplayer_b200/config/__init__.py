"""Typed configurations and the architecture registry."""
from .registry import (
    ArchitectureConfig, config_class_for, config_from_dict, known_architectures, load_config,
    register_architecture, unregister_architecture,
)
from .llama import LlamaConfig

__all__ = [
    "ArchitectureConfig", "LlamaConfig", "config_class_for", "config_from_dict",
    "known_architectures", "load_config", "register_architecture", "unregister_architecture",
]
