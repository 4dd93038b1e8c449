from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .lfm2 import ConfigError, Lfm2Config
from .registry import (Architecture, UnknownArchitecture, architecture_name, architectures,
                       load_config, lookup, read_config_json, register_architecture)

__all__ = [
    "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "ConfigError", "Lfm2Config",
    "Architecture", "UnknownArchitecture", "architecture_name", "architectures", "load_config",
    "lookup", "read_config_json", "register_architecture",
]
