"""Weights: sources of tensors by name, the strict name/shape check, random model folders."""

from .source import (DictSource, ParamSpec, RandomSource, SafetensorsSource, TiedWeightError, WeightError,
                     WeightSource, check_names_and_shapes, stored_dtype_policy)
from .random import random_tensors, write_random_model

__all__ = ["DictSource", "ParamSpec", "RandomSource", "SafetensorsSource", "TiedWeightError", "WeightError", "WeightSource",
           "check_names_and_shapes", "stored_dtype_policy", "random_tensors", "write_random_model"]
