from . import qwen3  # noqa: F401  (registers the architecture)
from .decoder import DecoderModel
from .loading import load_model, random_model

__all__ = ["DecoderModel", "load_model", "random_model"]
