"""Models assembled from parts. ``build_model`` turns a typed configuration into a ``Model``;
``load_model`` reads a model folder (``config.json`` chooses the architecture)."""

from __future__ import annotations

from typing import Dict, Union

import torch

from ..config import ModelConfig, ModelSpec, load_config
from ..weights.source import ParamSpec, SafetensorsSource, WeightSource
from .model import Model


def build_model(config: Union[ModelConfig, ModelSpec]) -> Model:
    return Model(config if isinstance(config, ModelSpec) else config.model_spec())


def expected_params(spec: ModelSpec) -> Dict[str, ParamSpec]:
    return Model(spec).expected_params()


def load_model(model_dir: str, device: Union[str, torch.device] = "cuda:0", dtype: torch.dtype = torch.bfloat16):
    """(config, model) of a folder holding config.json and *.safetensors."""
    config = load_config(model_dir)
    model = build_model(config)
    source = SafetensorsSource(model_dir)
    try:
        model.load(source, torch.device(device), dtype)
    finally:
        source.close()
    return config, model


__all__ = ["Model", "build_model", "expected_params", "load_model"]
