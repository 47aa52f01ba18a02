from .engine import EngineConfig, parse_dtype
from .llama import LlamaConfig
from .model import ConfigError, LayerSpec, ModelConfig, PartSpec, PlanEntry

__all__ = ["EngineConfig", "parse_dtype", "LlamaConfig", "ConfigError", "LayerSpec",
           "ModelConfig", "PartSpec", "PlanEntry"]
