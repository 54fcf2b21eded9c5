from .llama import ConfigError, LlamaConfig, RopeScaling
from .ropovik import RopovikConfig
from .senupel import SenupelConfig
from .zotolix import ZotolixConfig
from .registry import (Architecture, find_architecture, read_config_json, read_model_config,
                       register_architecture, registered_architectures, unregister_architecture)

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "RopovikConfig", "SenupelConfig", "ZotolixConfig", "Architecture", "find_architecture",
           "read_config_json", "read_model_config", "register_architecture",
           "registered_architectures", "unregister_architecture"]
