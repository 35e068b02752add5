"""Typed configurations, the model description they turn into, and the architecture registry."""
from .registry import (Architecture, architectures, load_config, read_config_json, register_architecture,
                       resolve_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .qwen3 import Qwen3Config, parse_qwen3_config, qwen3_spec

__all__ = ["Architecture", "architectures", "load_config", "read_config_json", "register_architecture",
           "resolve_architecture", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
           "parse_qwen3_config", "qwen3_spec"]
