from . import llama  # noqa: F401  (registers the architecture)
from .decoder import DecoderModel, expected_tensors
from .loading import load_model

__all__ = ["DecoderModel", "expected_tensors", "load_model"]
