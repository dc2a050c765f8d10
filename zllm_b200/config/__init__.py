from .model_config import LlamaConfig, RopeScaling, read_config_json
from .engine_config import EngineConfig
from .registry import (architecture, architecture_of, known_architectures,
                       register_architecture, ArchEntry)

__all__ = ["LlamaConfig", "RopeScaling", "read_config_json", "EngineConfig", "architecture",
           "architecture_of", "known_architectures", "register_architecture", "ArchEntry"]
