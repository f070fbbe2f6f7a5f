from .base import ConfigError, read_config_json
from .gpt2 import GPT2Config
from .registry import (Architecture, known_architectures, load_config,
                       register_architecture, resolve_architecture)

__all__ = ["ConfigError", "read_config_json", "GPT2Config", "Architecture",
           "known_architectures", "load_config", "register_architecture",
           "resolve_architecture"]
