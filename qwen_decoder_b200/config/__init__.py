from .model_config import ConfigError, Qwen2Config, read_config_json, write_config_json
from .registry import (
    PART_KINDS, config_from_dict, create_part, describe_model, known_architectures, load_config,
    lookup_architecture, register_architecture, register_part, unregister_architecture,
    unregister_part,
)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from . import qwen2 as _qwen2  # registers Qwen2ForCausalLM

__all__ = [
    "ConfigError", "Qwen2Config", "read_config_json", "write_config_json", "PART_KINDS",
    "config_from_dict", "create_part", "describe_model", "known_architectures", "load_config",
    "lookup_architecture", "register_architecture", "register_part", "unregister_architecture",
    "unregister_part", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry",
]
