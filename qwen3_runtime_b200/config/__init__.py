from .engine_config import EngineConfig, canonical_dtype
from .logesun_config import LogesunConfig
from .medilix_config import MedilixConfig
from .puladra_config import PuladraConfig
from .tabisun_config import TabisunConfig
from .model_config import ConfigError, Qwen3Config
from .registry import (
    Architecture,
    architecture_for_config,
    default_architecture,
    load_config,
    read_config_json,
    register_architecture,
    registered_architectures,
    resolve_architecture,
    unregister_architecture,
)
from .spec import LayerRun, ModelSpec, PartSpec

__all__ = [
    "Architecture",
    "architecture_for_config",
    "default_architecture",
    "ConfigError",
    "EngineConfig",
    "LayerRun",
    "LogesunConfig",
    "MedilixConfig",
    "ModelSpec",
    "PartSpec",
    "PuladraConfig",
    "Qwen3Config",
    "TabisunConfig",
    "canonical_dtype",
    "load_config",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]
