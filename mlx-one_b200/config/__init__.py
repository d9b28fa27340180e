from .base import ConfigError
from .farorax import FaroraxConfig
from .galarax import GalaraxConfig
from .lamisun import LamisunConfig
from .tirudra import TirudraConfig
from .lfm2 import Lfm2Config
from .registry import (Architecture, architecture_key, architecture_names, get_architecture, read_config,
                       register_architecture, unregister_architecture)

__all__ = ["ConfigError", "FaroraxConfig", "GalaraxConfig", "LamisunConfig", "Lfm2Config", "TirudraConfig", "Architecture", "architecture_key",
           "architecture_names",
           "get_architecture", "read_config", "register_architecture",
           "unregister_architecture"]
