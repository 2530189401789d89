from .base import ConfigError, ModelConfig, read_json
from .generation import GenerationConfig
from .qwen3 import Qwen3Config
from .suvazen import SuvazenConfig
from .sonalorn import SonalornConfig
from .zutazen import ZutazenConfig
from .mananex import MananexConfig
from .registry import (Architecture, known_architectures, load_config, register_architecture,
                       resolve_architecture, unregister_architecture)

__all__ = ["ConfigError", "ModelConfig", "GenerationConfig", "Qwen3Config", "SuvazenConfig", "SonalornConfig", "ZutazenConfig", "MananexConfig", "Architecture",
           "known_architectures", "load_config", "register_architecture",
           "resolve_architecture", "unregister_architecture", "read_json"]
