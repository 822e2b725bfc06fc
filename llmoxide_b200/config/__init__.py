"""Typed configuration, the architecture registry and the part-level model
description that the rest of the package reads."""

from .qwen3 import Qwen3Config
from .registry import architectures, config_class, read_config, register_architecture
from .spec import BlockSpec, LayerCall, ModelSpec, PartSpec, TensorSpec, default_schedule

register_architecture("Qwen3ForCausalLM", Qwen3Config)

__all__ = [
    "Qwen3Config", "architectures", "config_class", "read_config", "register_architecture",
    "BlockSpec", "LayerCall", "ModelSpec", "PartSpec", "TensorSpec", "default_schedule",
]
