"""Configuration: architecture-neutral specs, family configs, and the architecture registry."""
from .specs import (AttentionSpec, ConfigError, GatedMLPSpec, LayerSpec, ModelSpec,
                    NameLayout, NormSpec, RopeSpec, ScheduleEntry, ScoreSpec)
from .qwen3 import Qwen3Config
from .registry import (family_for, load_config, parse_config, read_config_json,
                       register_architecture, registered_architectures)

__all__ = [
    "AttentionSpec", "ConfigError", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NameLayout",
    "NormSpec", "RopeSpec", "ScheduleEntry", "ScoreSpec", "Qwen3Config", "family_for", "load_config",
    "parse_config", "read_config_json", "register_architecture", "registered_architectures",
]
