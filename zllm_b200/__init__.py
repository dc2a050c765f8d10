"""zllm_b200: a small, whole inference engine for the dense Llama decoder on one B200."""
from .errors import (BackendError, ConfigError, MemoryError_, ModelError, RequestError, ZllmError)

__version__ = "0.1.0"
__all__ = ["BackendError", "ConfigError", "MemoryError_", "ModelError", "RequestError", "ZllmError"]
