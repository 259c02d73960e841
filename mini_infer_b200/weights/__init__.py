"""Weights: safetensors I/O, binding by name, random-weights mode."""

from .loader import TensorSource, WeightLoadError, bind_state_dict, check_names, load_weights, to_engine_dtype  # noqa: F401
from .random_init import bind_random, random_state_dict, random_tensor, write_random_model  # noqa: F401
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401
