from .batch import SequenceSlice, StepBatch, build_batch
from .step import StepFunction

__all__ = ["SequenceSlice", "StepBatch", "build_batch", "StepFunction"]
