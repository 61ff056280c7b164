"""Typed configuration, the architecture registry and the named shapes."""
from .model_spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen2 import ARCHITECTURE as QWEN2_ARCHITECTURE
from .qwen2 import MODEL_TYPE as QWEN2_MODEL_TYPE
from .qwen2 import Qwen2Config, build_qwen2_spec, read_config_json
from .registry import (Architecture, register_architecture, registered_architectures, resolve,
                       spec_from_config_dict, unregister_architecture)
from .shapes import named_shape, shape_names

register_architecture(
    Architecture(QWEN2_ARCHITECTURE, QWEN2_MODEL_TYPE, Qwen2Config, build_qwen2_spec), replace=True)

__all__ = [
    "Architecture", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config", "ScheduleEntry",
    "build_qwen2_spec", "named_shape", "read_config_json", "register_architecture",
    "registered_architectures", "resolve", "shape_names", "spec_from_config_dict", "unregister_architecture",
]
