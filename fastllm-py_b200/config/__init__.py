from .base import ConfigError, read_raw_config
from .engine import EngineConfig, canonical_dtype
from .llama import LinearRopeScaling, LlamaConfig
from .tigitar import TigitarConfig
from .lasonex import LasonexConfig
from .sakusun import SakusunConfig
from .saberax import SaberaxConfig
from .registry import (Architecture, architecture_names, architecture_of, load_config,
                       register_architecture)

__all__ = [
    "ConfigError", "read_raw_config", "EngineConfig", "canonical_dtype", "LinearRopeScaling",
    "LlamaConfig", "TigitarConfig", "LasonexConfig", "SakusunConfig", "SaberaxConfig", "Architecture", "architecture_names", "architecture_of", "load_config",
    "register_architecture",
]
