from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (Architecture, register_architecture, registered_architectures,
                       resolve_architecture)
from .qwen3 import Qwen3Config
from .kefetar import KefetarConfig
from .mukenex import MukenexConfig
from .torinex import TorinexConfig
from .lufizen import LufizenConfig

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Architecture",
           "register_architecture", "registered_architectures", "resolve_architecture",
           "Qwen3Config", "KefetarConfig", "MukenexConfig", "TorinexConfig", "LufizenConfig"]
