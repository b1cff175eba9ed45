"""Weights: the safetensors container, loading by tensor name, random models."""

from .loader import WeightsError, load_model  # noqa: F401
from .random_init import load_random_model, write_random_model  # noqa: F401
from .safetensors_io import SafetensorsFile, open_model_files, write_safetensors  # noqa: F401
