"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` without biases
(src/llm_pipeline/models/qwen3/custom_builder.py:193-207; the activation is SiLU whatever
``hidden_act`` says, :204). Gate and up are one matrix product against [gate; up]."""

from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from ..ops.linear import PendingProduct, gate_up_swiglu, linear, pending_product
from ..weights.source import ParamSpec
from .base import FeedForward, TensorGetter
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int):
        self.prefix, self.hidden_size, self.intermediate_size = prefix, int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        return {f"{p}.gate_proj.weight": ParamSpec((I, H)), f"{p}.up_proj.weight": ParamSpec((I, H)),
                f"{p}.down_proj.weight": ParamSpec((H, I))}

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_gate_up = torch.cat([get(f"{p}.gate_proj.weight", "matrix"), get(f"{p}.up_proj.weight", "matrix")],
                                   dim=0).contiguous()
        self.w_down = get(f"{p}.down_proj.weight", "matrix").contiguous()

    takes_scaled_rows = True             # x goes straight into gate_up_swiglu() or linear()

    def forward(self, x, ctx):
        out, bias = self.forward_deferred(x, ctx)
        return (out.value() if isinstance(out, PendingProduct) else out), bias

    def forward_deferred(self, x, ctx):
        act = gate_up_swiglu(x, self.w_gate_up)          # the few rows of a decode step: product and activation in one kernel
        if act is None:
            gate_up = linear(x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
            kernels.swiglu(gate_up, act)
        return pending_product(act, self.w_down), None
