from .model_config import ConfigError, ModelConfig, Qwen2Config, read_config_json
from .registry import (
    Architecture,
    parse_config,
    register_architecture,
    registered_architectures,
    resolve_architecture,
)

__all__ = [
    "Architecture",
    "ConfigError",
    "ModelConfig",
    "Qwen2Config",
    "parse_config",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
]
