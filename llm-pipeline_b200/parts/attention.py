"""Grouped-query causal attention over the paged cache, as a mixer.

src/llm_pipeline/models/qwen3/custom_builder.py:110-190: q/k/v projections (biases by
``attention_bias``), RMSNorm over each head of q and k (:129-130), rotary on q and k (:133-134),
keys and values appended to the cache (:137-141: k after norm and rotary, v as projected), each
key/value head shared by ``num_heads // num_kv_heads`` consecutive query heads (:101-108), scores
scaled by ``head_dim ** -0.5`` after the product (:148), causal mask (:154-160), float32 softmax
(:179), weighted sum and output projection (:183-188).

The three projections are one matrix product against the row-wise concatenation [q; k; v] of
their weights; one kernel then applies bias, head norms and rotation and writes k and v to the
request's pages; the attention kernel reads all keys and values from pages, this step's included.
``window`` (None: every earlier key) and ``kv_shared`` (read the pages another execution wrote;
no k/v projection of its own) are parameters that Qwen3 leaves at None/False."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import KVPagesSpec
from ..ops import kernels
from ..ops.linear import PendingProduct, linear, pending_product
from ..weights.source import ParamSpec
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("attention")
class PagedAttention(Mixer):
    graph_safe = True      # a step only writes this step's keys and values: repeating it changes nothing

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, bias: bool = False, qk_norm: bool = True, qk_norm_eps: float = 1e-6,
                 window: Optional[int] = None, position: Optional[str] = "rope", rotary_dim: Optional[int] = None,
                 kv_shared: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"the attention kernels take head sizes that are multiples of 16 in 16..256, got {head_dim}")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale, self.bias, self.qk_norm, self.qk_norm_eps = float(scale), bool(bias), bool(qk_norm), float(qk_norm_eps)
        self.window, self.position, self.kv_shared = window, position, bool(kv_shared)
        self.rotary_dim = (head_dim if rotary_dim is None else int(rotary_dim)) if position else 0
        self.q_size, self.kv_size = num_heads * head_dim, num_kv_heads * head_dim
        self.tokens_per_tile: Optional[int] = None
        self.max_key_segments = 1            # items that may share a tile's keys in the kernel for these sizes
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = None

    # -- what it asks of the cache --------------------------------------------------------
    def cache_spec(self) -> Optional[KVPagesSpec]:
        return KVPagesSpec(self.num_kv_heads, self.head_dim, self.window)

    # -- weights ---------------------------------------------------------------------------
    def _projections(self):
        return ("q_proj",) if self.kv_shared else ("q_proj", "k_proj", "v_proj")

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H = self.prefix, self.hidden_size
        sizes = {"q_proj": self.q_size, "k_proj": self.kv_size, "v_proj": self.kv_size}
        specs = {f"{p}.{n}.weight": ParamSpec((sizes[n], H)) for n in self._projections()}
        specs[f"{p}.o_proj.weight"] = ParamSpec((H, self.q_size))
        if self.bias:
            for n in self._projections():
                specs[f"{p}.{n}.bias"] = ParamSpec((sizes[n],), role="vector")
            specs[f"{p}.o_proj.bias"] = ParamSpec((H,), role="vector")
        if self.qk_norm:
            specs[f"{p}.q_norm.weight"] = ParamSpec((self.head_dim,), role="vector", init="norm")
            if not self.kv_shared:
                specs[f"{p}.k_norm.weight"] = ParamSpec((self.head_dim,), role="vector", init="norm")
        return specs

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_qkv = torch.cat([get(f"{p}.{n}.weight", "matrix") for n in self._projections()], dim=0).contiguous()
        self.w_o = get(f"{p}.o_proj.weight", "matrix").contiguous()
        if self.bias:
            parts = [get(f"{p}.{n}.bias", "vector") for n in self._projections()]
            kind = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
            self.b_qkv = torch.cat([t.to(kind) for t in parts]).contiguous()
            self.b_o = get(f"{p}.o_proj.bias", "vector").contiguous()
        if self.qk_norm:
            self.q_norm = get(f"{p}.q_norm.weight", "vector").contiguous()
            self.k_norm = self.q_norm if self.kv_shared else get(f"{p}.k_norm.weight", "vector").contiguous()
            if self.k_norm.dtype != self.q_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    # -- one step --------------------------------------------------------------------------
    takes_scaled_rows = True             # x goes straight into linear()

    def forward(self, x, ctx, cache: LayerCache):
        out, bias = self.forward_deferred(x, ctx, cache)
        return (out.value() if isinstance(out, PendingProduct) else out), bias

    def forward_deferred(self, x, ctx, cache: LayerCache):
        if cache.pages is None or cache.group is None:
            raise RuntimeError("the attention mixer needs the pages of its cache")
        page_size = cache.pages.shape[3]
        if self.tokens_per_tile is None:
            self.tokens_per_tile = kernels.tokens_per_attention_tile(self.num_heads, self.num_kv_heads, x.dtype,
                                                                     self.head_dim, page_size)
            self.max_key_segments = kernels.attention_max_segments(self.num_heads, self.num_kv_heads, x.dtype,
                                                                   self.head_dim, page_size)
        qkv = linear(x, self.w_qkv)
        cos = sin = None
        if self.rotary_dim:
            cos, sin = ctx.position_tables[self.position]
        writes = cache.writes and not self.kv_shared
        kernels.qkv_post(qkv, self.num_heads, 0 if self.kv_shared else self.num_kv_heads, self.head_dim,
                         bias=self.b_qkv, q_weight=self.q_norm, k_weight=self.k_norm, eps=self.qk_norm_eps,
                         cos=cos, sin=sin, rotary_dim=self.rotary_dim,
                         slots=ctx.slot_mapping[cache.group] if writes else None,
                         pages=cache.pages if writes else None, page_size=page_size)
        out = torch.empty((ctx.num_tokens, self.q_size), dtype=x.dtype, device=x.device)
        ctx.attention(self, qkv, out, cache)
        return pending_product(out, self.w_o), self.b_o
