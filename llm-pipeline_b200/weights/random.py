"""Random-weights mode: write a model folder (``config.json`` and ``model.safetensors``) from a
configuration and a seed. The reference has no such feature; its tests rely on
``torch.manual_seed`` and the default initialisers of its modules
(src/llm_pipeline/testing/unit/test_qwen3_models.py:77-160)."""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Union

import torch

from ..config import ModelConfig, resolve_config
from .source import ParamSpec, RandomSource


def expected_params_of(config: ModelConfig) -> Dict[str, ParamSpec]:
    from ..models import expected_params

    return expected_params(config.model_spec())


def random_tensors(config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                   device: str = "cpu") -> RandomSource:
    return RandomSource(expected_params_of(config), seed, std=std, dtype=dtype, device=device)


def write_random_model(config: Union[ModelConfig, Dict[str, Any]], seed: int, out_dir: str,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02) -> str:
    """Create ``out_dir`` with ``config.json`` and ``model.safetensors`` and return its path."""
    from safetensors.torch import save_file

    config_json = config if isinstance(config, dict) else config.to_json()
    typed = resolve_config(config_json) if isinstance(config, dict) else config
    source = random_tensors(typed, seed, dtype=dtype, std=std)
    os.makedirs(out_dir, exist_ok=True)
    tensors = {name: source.get(name).contiguous() for name in source.names()}
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    out_json = dict(config_json)
    out_json.setdefault("architectures", [typed.architecture])
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(out_json, f, indent=1)
    return out_dir
