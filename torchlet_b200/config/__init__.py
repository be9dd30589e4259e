from .engine import EngineConfig, ceil_div
from .registry import (
    architecture_name,
    config_class_for,
    config_from_dict,
    known_architectures,
    load_config,
    register_architecture,
)
from .spec import LayerSpec, ModelSpec, NormSlot, PartSpec, ScheduleEntry
from .qwen2 import Qwen2Config
from .dodonex import DodonexConfig
from .numuzen import NumuzenConfig
from .fusolix import FusolixConfig
from .kilatar import KilatarConfig

__all__ = [
    "DodonexConfig",
    "EngineConfig",
    "FusolixConfig",
    "KilatarConfig",
    "LayerSpec",
    "ModelSpec",
    "NumuzenConfig",
    "NormSlot",
    "PartSpec",
    "Qwen2Config",
    "ScheduleEntry",
    "architecture_name",
    "ceil_div",
    "config_class_for",
    "config_from_dict",
    "known_architectures",
    "load_config",
    "register_architecture",
]
