from .golulix import GolulixConfig
from .llama import ConfigError, LlamaConfig, RopeScaling
from .nekotar import NekotarConfig
from .rudazen import RudazenConfig
from .samulorn import SamulornConfig
from .registry import (architectures, config_from_dict, load_config,
                       register_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

__all__ = ["ConfigError", "GolulixConfig", "LlamaConfig", "NekotarConfig", "RudazenConfig", "SamulornConfig", "RopeScaling", "architectures",
           "config_from_dict", "load_config", "register_architecture",
           "LayerSpec", "ModelSpec", "PartSpec", "RunEntry"]
