"""One error family for the whole engine.

Mirrors the reference's single enum (zllm src/error.rs:3-27: Config / Model /
Memory / Backend / ...): every failure a caller can act on is one of these, and
each message names the thing that is wrong (the key, the tensor, the size).
"""


class ZllmError(Exception):
    """Base of every error this package raises on purpose."""


class ConfigError(ZllmError):
    """A configuration key is missing, unknown or has an unusable value."""


class ModelError(ZllmError):
    """A model folder or its tensors cannot be used (missing, unexpected, wrong shape)."""


class MemoryError_(ZllmError):
    """The cache pool cannot supply what was asked (pages or slots exhausted)."""


class BackendError(ZllmError):
    """The CUDA extension is missing, failed to build, or a kernel refused its sizes."""


class RequestError(ZllmError):
    """A request cannot be admitted (empty prompt, too long, unknown id)."""
