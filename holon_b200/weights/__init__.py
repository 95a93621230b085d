"""Weights: sources (a folder of safetensors, or seeded random tensors under the same names) and the loader."""
from .loader import NameMap, WeightError, load_weights
from .source import RandomSource, SafetensorsSource, write_model_folder

__all__ = ["NameMap", "RandomSource", "SafetensorsSource", "WeightError", "load_weights", "write_model_folder"]
