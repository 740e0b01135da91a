"""Model files: the safetensors container, the by-name loader and the random-weights mode."""
from .safetensors_io import SafetensorsFile, write_safetensors
from .loader import COMPUTE_DTYPES, canonical_dtype, load_parameters, random_parameters
from .random_init import normal_values, random_tensors, write_random_model

__all__ = ["SafetensorsFile", "write_safetensors", "COMPUTE_DTYPES", "canonical_dtype", "load_parameters",
           "random_parameters", "normal_values", "random_tensors", "write_random_model"]
