from .llama import ConfigError, LlamaConfig, RopeScaling
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec, check_schedule
from .registry import (Architecture, architecture, known_architectures, read_config_json,
                       register_architecture, resolve, resolve_model_dir)
from .engine import EngineConfig

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "LayerSpec", "ModelSpec", "PartSpec",
           "RunSpec", "check_schedule", "Architecture", "architecture", "known_architectures",
           "read_config_json", "register_architecture", "resolve", "resolve_model_dir", "EngineConfig"]
