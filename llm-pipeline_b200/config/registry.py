"""One registry from an architecture's name (``config.json["architectures"][0]``) to its typed
configuration. The reference keeps a dictionary from a name to an entry with required keys and a
``register`` call that checks them (src/llm_pipeline/core/registry.py:50-62,102-109); its engine
hard-wires the Qwen3 factory (src/llm_pipeline/inference/qwen3_engine.py:175). Here the entry
is the configuration class, and the model is built from the ``ModelSpec`` that class produces."""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Type

from .base import ModelConfig

_ARCHITECTURES: Dict[str, Type[ModelConfig]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig]) -> None:
    if not (isinstance(config_cls, type) and issubclass(config_cls, ModelConfig)):
        raise TypeError(f"{config_cls!r} is not a ModelConfig subclass")
    _ARCHITECTURES[name] = config_cls


def supported_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(config_json: Dict[str, Any]) -> str:
    names = config_json.get("architectures") or []
    if names:
        return str(names[0])
    model_type = config_json.get("model_type")
    for name, cls in _ARCHITECTURES.items():
        if model_type is not None and getattr(cls, "model_type", None) == model_type:
            return name
    raise ValueError("config.json names no architecture: it has neither 'architectures' nor a known "
                     f"'model_type' (supported: {supported_architectures()})")


def resolve_config(config_json: Dict[str, Any]) -> ModelConfig:
    name = architecture_name(config_json)
    if name not in _ARCHITECTURES:
        raise ValueError(f"unsupported architecture {name!r}; supported: {supported_architectures()}")
    return _ARCHITECTURES[name].from_json(config_json)


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir!r}")
    with open(path) as f:
        return resolve_config(json.load(f))
