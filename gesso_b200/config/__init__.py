"""Typed configuration and the architecture registry."""
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .registry import (architecture_name, known_architectures, parse_strict_json, read_config,
                       register_architecture, spec_from_config, spec_from_dir,
                       unregister_architecture)
from .lfm2 import Lfm2Config, effective_ff_dim

__all__ = [
    "BlockSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule",
    "architecture_name", "known_architectures", "parse_strict_json", "read_config",
    "register_architecture", "spec_from_config", "spec_from_dir", "unregister_architecture",
    "Lfm2Config", "effective_ff_dim",
]
