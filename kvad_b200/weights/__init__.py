"""Weights: safetensors by tensor name, one audit, and a random-weights mode."""
from .safetensors_io import Checkpoint, SafetensorsError, TensorEntry, write_safetensors
from .source import SPELLINGS, TensorRequest, WeightSource, WeightsError, collapse
from .random_init import write_random_model

__all__ = [
    "Checkpoint", "SafetensorsError", "TensorEntry", "write_safetensors", "SPELLINGS",
    "TensorRequest", "WeightSource", "WeightsError", "collapse", "write_random_model",
]
