from .base import ConfigError, ModelConfig, read_config_json
from .presets import load_preset, preset_names
from .qwen3 import Qwen3Config
from .registry import (Architecture, config_from_dict, get_architecture, load_config,
                       register_architecture, registered_architectures,
                       unregister_architecture)

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "Architecture", "config_from_dict",
           "get_architecture", "load_config", "load_preset", "preset_names", "read_config_json", "register_architecture",
           "registered_architectures", "unregister_architecture"]
