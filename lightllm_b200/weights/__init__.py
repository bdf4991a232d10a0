from .loader import WeightError, WeightSpec, check_against, dedup_specs, load_checkpoint_tensors, target_dtype
from .random_init import draw_tensor, random_tensors, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, TensorInfo, save_file

__all__ = [
    "WeightError", "WeightSpec", "check_against", "dedup_specs", "load_checkpoint_tensors", "target_dtype",
    "draw_tensor", "random_tensors", "write_random_model",
    "Checkpoint", "SafetensorsError", "SafetensorsFile", "TensorInfo", "save_file",
]
