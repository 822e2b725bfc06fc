"""llmoxide_b200: a small, whole generation library for one GPU (NVIDIA B200,
sm_100a): typed configuration and an architecture registry, safetensors
weights, layers put together from parts, a paged cache with a slot per
sequence, one step function, a generation loop with sampling, and trace
replay.  Everything between a request's tokens and its next token."""

from .config import Qwen3Config, read_config, register_architecture
from .engine.engine import Engine, LoadOptions
from .engine.generate import Outcome, Request
from .errors import (CacheExhausted, CacheMisuse, CheckpointFormatError, ConfigError, ContextOverflow,
                     ExtensionMissing, KernelError, LlmoxideError, Unsupported, UnsupportedArch, WeightsError)
from .sampling.params import Sampling
from .session import Session
from .weights import write_model_folder

__all__ = [
    "Session", "Engine", "LoadOptions", "Request", "Outcome", "Sampling", "Qwen3Config", "read_config",
    "register_architecture", "write_model_folder", "LlmoxideError", "ConfigError", "UnsupportedArch",
    "Unsupported", "WeightsError", "CheckpointFormatError", "ContextOverflow", "CacheExhausted", "CacheMisuse",
    "ExtensionMissing", "KernelError",
]
