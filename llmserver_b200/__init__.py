"""llmserver_b200: a small, whole, single-GPU inference engine for B200 (sm_100a).

Everything between a request's tokens and its next token for the Qwen3 dense architecture:
typed configuration and architecture registry, weights by tensor name, layers put together from
parts, a paged cache manager, one step function for mixed batches, a continuous-batching scheduler,
sampling, hand-written CUDA kernels, a true 32-bit path and trace replay.
"""
from .config import Qwen3Config, UnsupportedModelError, WeightLoadError, read_config  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # heavier pieces are imported on first use so that configuration tools start quickly
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    if name in ("load_model", "random_model"):
        from . import models
        return getattr(models, name)
    raise AttributeError(name)
