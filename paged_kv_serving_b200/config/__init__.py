"""Typed configurations and the registries."""

from paged_kv_serving_b200.config.engine_config import DTYPES, EngineConfig
from paged_kv_serving_b200.config.model_config import CONFIG_FILE, ModelConfig
from paged_kv_serving_b200.config.registry import (
    architecture, known_architectures, known_parts, part, register_architecture, register_part,
)

__all__ = [
    "CONFIG_FILE", "DTYPES", "EngineConfig", "ModelConfig", "architecture", "known_architectures",
    "known_parts", "part", "register_architecture", "register_part",
]
