"""zllm_b200: a small, whole inference engine for the dense Llama decoder on one B200.

    from zllm_b200 import Engine, SamplingParams
    eng = Engine("path/to/model")                      # config.json + model.safetensors
    out = eng.generate([[1, 2, 3]], SamplingParams.greedy(max_tokens=16))
"""
from .errors import (BackendError, ConfigError, MemoryError_, ModelError, RequestError, ZllmError)
from .config import EngineConfig, LlamaConfig
from .sampling import SamplingParams
from .engine import Engine, ModelRunner, Session, StepEntry

__version__ = "0.1.0"
__all__ = ["BackendError", "ConfigError", "MemoryError_", "ModelError", "RequestError", "ZllmError",
           "EngineConfig", "LlamaConfig", "SamplingParams", "Engine", "ModelRunner", "Session", "StepEntry"]
