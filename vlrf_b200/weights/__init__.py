from .safetensors_io import WeightError, read_safetensors, write_safetensors
from .spec import CheckedWeights, TensorSpec, check_tensors, place
from .model_dir import open_model_dir, write_random_model

__all__ = ["WeightError", "read_safetensors", "write_safetensors", "CheckedWeights", "TensorSpec",
           "check_tensors", "place", "open_model_dir", "write_random_model"]
