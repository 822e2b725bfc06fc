"""Weights: safetensors by tensor name, checked against the model description,
and the random-weights mode."""

from .loader import check_checkpoint, load_checkpoint, target_dtype
from .random_init import random_tensors_on_device, write_model_folder
from .safetensors_io import SafetensorsFile, SafetensorsWriter, open_checkpoint, save_file

__all__ = [
    "check_checkpoint", "load_checkpoint", "target_dtype", "random_tensors_on_device",
    "write_model_folder", "SafetensorsFile", "SafetensorsWriter", "open_checkpoint", "save_file",
]
