from .model_config import ConfigError, ConfigReader, ModelConfig, architecture_name, read_config_json
from .model_spec import LayerSpec, ModelSpec, PartSpec, RunEntry, SubBlock
from .registry import (config_from_dict, known_architectures, load_config, model_spec_for,
                       part_class, register_architecture, register_part)

__all__ = [
    "ConfigError", "ConfigReader", "ModelConfig", "architecture_name", "read_config_json",
    "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "SubBlock",
    "config_from_dict", "known_architectures", "load_config", "model_spec_for",
    "part_class", "register_architecture", "register_part",
]
