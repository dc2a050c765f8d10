from .decoder import DecoderModel, Runtime, expected_tensors, optional_tensors, required_tensors
from . import llama  # noqa: F401  (registers LlamaForCausalLM)

__all__ = ["DecoderModel", "Runtime", "expected_tensors", "optional_tensors", "required_tensors"]
