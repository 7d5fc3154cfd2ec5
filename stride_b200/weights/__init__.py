from .loader import TensorDecl, WeightMismatchError, check_source, load_weights, target_dtype
from .safetensors_io import SafetensorsFile, WeightFileError, find_shards, save_file
from .sources import DictSource, RandomSource, SafetensorsSource, WeightSource

__all__ = ["TensorDecl", "WeightMismatchError", "check_source", "load_weights", "target_dtype", "SafetensorsFile",
           "WeightFileError", "find_shards", "save_file", "DictSource", "RandomSource", "SafetensorsSource", "WeightSource"]
