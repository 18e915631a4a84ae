from .base import (ConfigError, ModelConfig, architecture_of, architectures, config_from_dict,
                   load_config, lookup_architecture, register_architecture)
from .dizepel import DizepelConfig
from .gotulorn import GotulornConfig
from .konovik import KonovikConfig
from .lefulorn import LefulornConfig
from .llama import LlamaConfig, RopeScaling

__all__ = ["ConfigError", "ModelConfig", "DizepelConfig", "GotulornConfig", "KonovikConfig", "LefulornConfig", "LlamaConfig", "RopeScaling", "architecture_of", "architectures",
           "config_from_dict", "load_config", "lookup_architecture", "register_architecture"]
