"""Typed configurations and the registry from an architecture's name to its model."""
from .base import (ConfigError, ArchitectureConfig, ArchitectureEntry, register_architecture, find_architecture,
                   known_architectures, read_config_json, config_from_dict, config_from_dir)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ArchitectureConfig", "ArchitectureEntry", "register_architecture", "find_architecture",
           "known_architectures", "read_config_json", "config_from_dict", "config_from_dir",
           "Qwen3Config"]
