from .specs import BlockSpec, ConfigError, ModelSpec, PartSpec, RunStep
from .registry import (Architecture, architecture_name_of, get_architecture, known_architectures,
                       load_config, register_architecture)
from .qwen2 import Qwen2Config

register_architecture("Qwen2ForCausalLM", Qwen2Config, replace=True)

__all__ = ["BlockSpec", "ConfigError", "ModelSpec", "PartSpec", "RunStep", "Architecture",
           "architecture_name_of", "get_architecture", "known_architectures", "load_config",
           "register_architecture", "Qwen2Config"]
