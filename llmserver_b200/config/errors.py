"""Error types of configuration and loading."""


class UnsupportedModelError(ValueError):
    """The model folder describes something this engine does not run; the message says what.

    Same role as ``UnsupportedModelError`` in the reference (utils/architecture.py:19-20)."""


class WeightLoadError(ValueError):
    """model.safetensors does not match what the configuration declares; the message lists every
    missing tensor, every unexpected tensor and every tensor of a wrong shape or dtype family."""
