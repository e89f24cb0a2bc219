from .loader import (WeightError, check_names, load_checkpoint, random_tensor, random_weights,
                     storage_dtype, write_model_folder)
from .safetensors_io import (Checkpoint, SafetensorsError, SafetensorsFile, discover_weight_files,
                             write_safetensors)

__all__ = ["WeightError", "check_names", "load_checkpoint", "random_tensor", "random_weights",
           "storage_dtype", "write_model_folder", "Checkpoint", "SafetensorsError",
           "SafetensorsFile", "discover_weight_files", "write_safetensors"]
