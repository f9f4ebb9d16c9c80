from .dtypes import resolve_dtype
from .registry import (ModelConfig, config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen2 import Qwen2Config
from .presets import preset_config, preset_dict, preset_names

__all__ = [
    "resolve_dtype", "ModelConfig", "config_class_for", "config_from_dict", "load_config", "register_architecture",
    "registered_architectures", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen2Config",
    "preset_config", "preset_dict", "preset_names",
]
