"""RMSNorm fused with the residual add.

Formula of src/llm_pipeline/models/qwen3/custom_builder.py:53-58: in float32,
``weight * (x * rsqrt(mean(x^2) + eps))``, rounded once to the compute type. The residual adds of
custom_builder.py:244,250 are folded in: the addend left by the previous part is summed into the
float32 residual by the same kernel that normalises it."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import residual_product
from ..weights.source import ParamSpec
from .base import Norm, ResidualStream, TensorGetter
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, prefix: str, size: int, eps: float):
        self.prefix, self.size, self.eps = prefix, int(size), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {f"{self.prefix}.weight": ParamSpec((self.size,), role="vector", init="norm")}

    def load(self, get: TensorGetter) -> None:
        self.weight = get(f"{self.prefix}.weight", "vector").contiguous()

    def add_norm(self, stream: ResidualStream, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        count = rows.numel() if rows is not None else stream.residual.shape[0]
        out = torch.empty((count, self.size), dtype=ctx.dtype, device=stream.residual.device)
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out,
                            delta_bias=stream.pending_bias, rows=rows)
        if rows is None:
            stream.pending, stream.pending_bias = None, None
        return out

    def add_norm_deferred(self, stream: ResidualStream, ctx):
        """As ``add_norm`` for all rows, but a pending product of a decode step's few rows is added into the residual by
        its own kernel, which leaves the rows normalised but for their factors (``ScaledRows``) to the product after."""
        product = stream.take_pending_product()
        if product is None:
            return self.add_norm(stream, ctx)
        residual = stream.residual
        if product.accumulate:
            # many rows: the library's product adds itself into the residual, the norm kernel only reads it
            if not kernels.library_add_product(residual, product.x, product.weight):
                stream.add(product.value())
            return self.add_norm(stream, ctx)

        def finished() -> torch.Tensor:
            # for a consumer that cannot apply the factors: the norm of the residual as it now is
            out = torch.empty((residual.shape[0], self.size), dtype=ctx.dtype, device=residual.device)
            return kernels.add_rmsnorm(residual, None, self.weight, self.eps, out)

        return residual_product(product, residual, self.weight, self.eps, finished)
