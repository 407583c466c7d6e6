from .files import ConfigError, read_config_files
from .debuvik import DebuvikConfig
from .dezolorn import DezolornConfig
from .fubolix import FubolixConfig
from .sorizen import SorizenConfig
from .llama import Llama3RopeScaling, LlamaConfig
from .recipe import LayerSpec, ModelRecipe, PartSpec, Run
from .registry import Architecture, register_architecture, registered_architectures, resolve_architecture
from .engine import EngineConfig

__all__ = [
    "Architecture", "ConfigError", "DebuvikConfig", "DezolornConfig", "EngineConfig", "FubolixConfig", "LayerSpec", "Llama3RopeScaling", "LlamaConfig",
    "ModelRecipe", "PartSpec", "Run", "SorizenConfig", "read_config_files", "register_architecture",
    "registered_architectures", "resolve_architecture",
]
