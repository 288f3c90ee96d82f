from .loader import TensorSpec, WeightError, WeightSpec, check_and_select, load_weights
from .model_folder import write_model_folder
from .safetensors_io import SafetensorsError, read_file, read_folder, read_header, write_file

__all__ = [
    "SafetensorsError", "TensorSpec", "WeightError", "WeightSpec", "check_and_select", "load_weights",
    "read_file", "read_folder", "read_header", "write_file", "write_model_folder",
]
