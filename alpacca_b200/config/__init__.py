from .base import ConfigError, ModelConfig
from .buguzen import BuguzenConfig
from .lefatar import LefatarConfig
from .llama import LlamaConfig
from .sazepel import SazepelConfig
from .registry import (Architecture, config_from_dict, get_architecture, load_config,
                       register_architecture, registered_architectures, unregister_architecture)

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "LefatarConfig", "BuguzenConfig", "SazepelConfig", "Architecture", "config_from_dict",
           "get_architecture", "load_config", "register_architecture", "registered_architectures",
           "unregister_architecture"]
