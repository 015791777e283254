"""Typed configurations and the architecture registry."""
from .base import ConfigError, ModelConfig, read_config_json
from .qwen3 import Qwen3Config
from .tovalix import TovalixConfig, TovalixLayer
from .nufupel import NufupelConfig, NufupelLayer
from .nikonex import NikonexConfig, NikonexLayer
from .meropel import MeropelConfig, MeropelLayer
from .registry import (Architecture, config_from_dict, known_architectures, load_config, lookup_architecture,
                       register_architecture)
from . import meropel_model, nikonex_model, nufupel_model, qwen3_model, tovalix_model  # noqa: F401,E402  (register the architectures)

__all__ = ["Architecture", "ConfigError", "MeropelConfig", "MeropelLayer", "ModelConfig", "NikonexConfig", "NikonexLayer", "NufupelConfig", "NufupelLayer", "Qwen3Config", "TovalixConfig", "TovalixLayer", "config_from_dict", "known_architectures",
           "load_config", "lookup_architecture", "read_config_json", "register_architecture"]
