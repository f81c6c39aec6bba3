from .engine import EngineConfig, parse_dtype
from .bizetar import BizetarConfig
from .llama import LlamaConfig
from .vapelix import VapelixConfig
from .vomotar import VomotarConfig
from .model import ConfigError, LayerSpec, ModelConfig, PartSpec, PlanEntry

__all__ = ["EngineConfig", "parse_dtype", "BizetarConfig", "LlamaConfig", "VomotarConfig", "VapelixConfig", "ConfigError", "LayerSpec",
           "ModelConfig", "PartSpec", "PlanEntry"]
