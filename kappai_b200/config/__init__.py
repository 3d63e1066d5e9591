from .schema import (ConfigError, TypedConfig, cfg, PartSpec, LayerSpec, ScheduleEntry, ModelSpec,
                     read_config_json)
from .registry import (Architecture, register_architecture, unregister_architecture,
                       lookup_architecture, architecture_names, architecture_of,
                       config_from_dict, load_config)

__all__ = [
    "ConfigError", "TypedConfig", "cfg", "PartSpec", "LayerSpec", "ScheduleEntry", "ModelSpec",
    "read_config_json", "Architecture", "register_architecture", "unregister_architecture",
    "lookup_architecture", "architecture_names", "architecture_of", "config_from_dict", "load_config",
]
