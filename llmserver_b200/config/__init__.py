from .errors import UnsupportedModelError, WeightLoadError
from .spec import PartSpec, LayerSpec, ScheduleEntry, ModelSpec
from .registry import ARCHITECTURES, Architecture, register_architecture, architecture_of, read_config
from .qwen3 import Qwen3Config, FULL_ATTENTION, SLIDING_ATTENTION

__all__ = ["UnsupportedModelError", "WeightLoadError", "PartSpec", "LayerSpec", "ScheduleEntry", "ModelSpec",
           "ARCHITECTURES", "Architecture", "register_architecture", "architecture_of", "read_config",
           "Qwen3Config", "FULL_ATTENTION", "SLIDING_ATTENTION"]
