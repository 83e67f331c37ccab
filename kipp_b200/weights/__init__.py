from .loader import Checkpoint, WeightError, load_tensors, open_checkpoint, storage_dtype
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, write_safetensors
from .spec import INIT_INT, INIT_NEAR_ONE, INIT_NORMAL, TensorSpec

__all__ = ["Checkpoint", "WeightError", "load_tensors", "storage_dtype", "random_tensors", "write_random_model",
           "SafetensorsError", "open_checkpoint", "write_safetensors", "INIT_INT", "INIT_NEAR_ONE",
           "INIT_NORMAL", "TensorSpec"]
