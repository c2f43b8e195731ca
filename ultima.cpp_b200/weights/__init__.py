"""Weights: safetensors files read by tensor name, and seeded random model folders."""
from .safetensors_io import SafetensorsError, read_safetensors_header, open_safetensors, write_safetensors
from .spec import WeightSpec, WeightError
from .loader import check_weights, load_weights, storage_dtype
from .random_init import counter_fill, counter_normal, random_tensors, random_tensors_on_device, write_random_model

__all__ = ["check_weights", "SafetensorsError", "read_safetensors_header", "open_safetensors", "write_safetensors",
           "WeightSpec", "WeightError", "load_weights", "storage_dtype", "random_tensors", "random_tensors_on_device",
           "write_random_model", "counter_fill", "counter_normal"]
