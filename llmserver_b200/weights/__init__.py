from .declare import MATRIX, NORM, TABLE, WeightDecl, declared_weights
from .reader import CheckpointReader
from .loader import CheckpointSource, check_checkpoint
from .random_init import RandomSource, random_tensor, write_model_folder

__all__ = ["MATRIX", "NORM", "TABLE", "WeightDecl", "declared_weights", "CheckpointReader", "CheckpointSource",
           "check_checkpoint", "RandomSource", "random_tensor", "write_model_folder"]
