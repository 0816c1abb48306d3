"""Typed configurations and the architecture registry."""

from .engine_config import EngineConfig, resolve_dtype_name
from .model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .qwen2_config import ConfigError, Qwen2Config
from .fovudra_config import FovudraConfig
from .zelasun_config import ZelasunConfig
from .zururax_config import ZururaxConfig
from .zuzunex_config import ZuzunexConfig
from .registry import (
    Architecture,
    architecture_of,
    get_architecture,
    known_architectures,
    read_config,
    register_architecture,
    unregister_architecture,
)

__all__ = [
    "Architecture",
    "ConfigError",
    "EngineConfig",
    "FovudraConfig",
    "LayerCall",
    "LayerSpec",
    "ModelSpec",
    "PartSpec",
    "Qwen2Config",
    "ZelasunConfig",
    "ZururaxConfig",
    "ZuzunexConfig",
    "architecture_of",
    "get_architecture",
    "known_architectures",
    "read_config",
    "register_architecture",
    "resolve_dtype_name",
    "unregister_architecture",
]
