"""Rotary position encoding: the per-step cos/sin tables.

src/llm_pipeline/models/qwen3/custom_builder.py:269-288: ``inv_freq[j] = 1 / theta^(2j/d)``
(float32), angle = position * inv_freq, cos and sin of the angle times ``attention_scaling``
(1.0), all in float32. The tables are ``[tokens, rotary_dim / 2]`` because the reference's
``cat(freqs, freqs)`` repeats them; the mixer's kernel pairs entry j with j + rotary_dim/2
(custom_builder.py:85-99). The reference rounds the tables to the activations' type
(custom_builder.py:288); here they stay float32."""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import PositionEncoding
from .registry import register_position


@register_position("rotary")
class RotaryPositions(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix: str, rotary_dim: int, theta: float, scaling: float = 1.0):
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        self.prefix, self.rotary_dim, self.theta, self.scaling = prefix, int(rotary_dim), float(theta), float(scaling)
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).float() / self.rotary_dim
        self._inv_freq_cpu = 1.0 / (self.theta ** exponent)
        self._inv_freq = None

    def tables(self, ctx):
        if self._inv_freq is None or self._inv_freq.device != ctx.device:
            self._inv_freq = self._inv_freq_cpu.to(ctx.device)
        half = self.rotary_dim // 2
        cos = torch.empty((ctx.num_tokens, half), dtype=torch.float32, device=ctx.device)
        sin = torch.empty_like(cos)
        kernels.rope_tables(ctx.positions, self._inv_freq, self.scaling, cos, sin)
        return cos, sin
