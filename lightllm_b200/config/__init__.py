from .model_config import ConfigError, ModelConfig, Qwen2Config, read_config_json
from .model_spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (config_from_dict, known_architectures, load_config, model_spec_for,
                       part_class, register_architecture, register_part)

__all__ = [
    "ConfigError", "ModelConfig", "Qwen2Config", "read_config_json",
    "LayerSpec", "ModelSpec", "PartSpec", "RunEntry",
    "config_from_dict", "known_architectures", "load_config", "model_spec_for",
    "part_class", "register_architecture", "register_part",
]
