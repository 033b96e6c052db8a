from .base import (
    Architecture,
    ConfigError,
    ModelConfig,
    load_config,
    parse_config,
    read_config_json,
    register_architecture,
    registered_architectures,
    resolve_architecture,
    unregister_architecture,
)
from .engine import EngineConfig
from .gpt2 import GPT2Config
from .lebedra import LebedraConfig
from .porovik import PorovikConfig
from .fikevik import FikevikConfig
from .soporax import SoporaxConfig

__all__ = [
    "Architecture",
    "ConfigError",
    "EngineConfig",
    "GPT2Config",
    "LebedraConfig",
    "PorovikConfig",
    "FikevikConfig",
    "SoporaxConfig",
    "ModelConfig",
    "load_config",
    "parse_config",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]
