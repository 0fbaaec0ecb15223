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
no k/v projection of its own) are parameters that Qwen3 leaves at None/False.

The mixer owns everything about its kernels: which one a step's shape gets (``graph_key``, ``attend``), the policy
constants (``AttentionPolicy``) and the work list of the general kernel. The step function only asks every mixer for
its ``graph_key`` when it keys a captured decode step."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.spec import KVPagesSpec
from ..ops import kernels
from ..ops.linear import PendingProduct, linear, pending_product
from ..weights.source import ParamSpec
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


class AttentionPolicy:
    """Which kernel an attention step takes and how its work is listed. Class attributes, so that tests can force a
    path at tiny sizes."""

    # Keys that one of the single-token requests at the front of a mixed step must see before they get a launch of the
    # decode kernel to themselves. Below that their tiles run beside the prompt portions' tiles of the general kernel
    # and end before them (8 requests of 8,192 keys beside a 2,048-token portion of Qwen3-8B: 29.8 ms per step either
    # way); above it the one block per key/value head that walks such a context alone is what the step waits for
    # (one request of 32,768 keys: 43.8 ms, with the decode kernel 26.9 ms).
    SPLIT_DECODE_MIN_CONTEXT = 16384
    # Key tiles (of KEY_TILE keys) that an item of the general attention kernel keeps at least when a tile's keys are
    # shared among items: below 2,048 keys an item's fixed cost and the adding up of sums outweigh the better balance.
    SPLIT_KEYS_MIN_TILES = 16
    # Up to one block per SM the work list shares tiles among items, and then aims at four blocks per SM: two rounds
    # of the two blocks that an SM holds. Qwen3-8B heads, 512 new tokens over 32,768 keys (128 blocks): 551 us whole,
    # 370 us as 4 items a tile (3 items: 432, 5 items: 410); 64 new tokens over 65,536 keys: 1,092 against 169 us;
    # 1,024 new tokens over 16,384 keys (256 blocks) gain nothing from it.
    SPLIT_KEYS_BELOW = 1.0
    SPLIT_KEYS_FILL = 4
    KEY_TILE = 128

    @classmethod
    def plan_items(cls, starts: List[int], q_lens: List[int], tokens_per_tile: int, first_request: int,
                   max_segments: int, num_kv_heads: int, sms: int):
        """The work list of the general attention kernel for the requests from ``first_request`` on, as host lists
        (request, first token, item of its tile | items << 8, first place of the tile) and the number of places, for a
        GPU of ``sms`` SMs. A tile is ``tokens_per_tile`` consecutive new tokens of a request. Where the kernel can share
        a tile's keys among items (``max_segments`` > 1) and the tiles are too few to give every SM a block (few new
        tokens over long contexts), a tile comes as several consecutive items, each with an equal share of its keys and
        at least ``SPLIT_KEYS_MIN_TILES`` key tiles."""
        found = []
        for r in range(first_request, len(q_lens)):
            n = q_lens[r]
            before = starts[r]
            for t in range(0, n, tokens_per_tile):
                found.append((before + min(t + tokens_per_tile, n), r, t))
        segments = [1] * len(found)
        blocks = len(found) * num_kv_heads
        if max_segments > 1 and blocks <= cls.SPLIT_KEYS_BELOW * sms:
            key_tiles = [-(-f[0] // cls.KEY_TILE) for f in found]
            want = cls.SPLIT_KEYS_FILL * sms // blocks       # never more than SPLIT_KEYS_FILL full rounds of blocks
            segments = [max(1, min(max_segments, want, k // cls.SPLIT_KEYS_MIN_TILES)) for k in key_tiles]
            if sum(n for n in segments if n > 1) * num_kv_heads > kernels.ATTENTION_MAX_PLACES:
                segments = [1] * len(found)
        # in the order of the keys an item sees: the kernels start the last item first, the longest blocks lead
        order = sorted(range(len(found)), key=lambda i: (found[i][0] / segments[i], found[i][1], found[i][2]))
        req, tok0, seg, slot = [], [], [], []
        places = 0
        for i in order:
            for k in range(segments[i]):
                req.append(found[i][1])
                tok0.append(found[i][2])
                seg.append(k | segments[i] << 8)
                slot.append(places if segments[i] > 1 else 0)
            if segments[i] > 1:
                places += segments[i]
        return req, tok0, seg, slot, places


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
        self.attend(ctx, qkv, out, cache)
        return pending_product(out, self.w_o), self.b_o

    # -- which kernel a step takes -----------------------------------------------------------
    def graph_key_group(self):
        return ("attention", self.num_kv_heads)            # the choice below depends on nothing else of the mixer

    def captured_context_limit(self) -> int:
        return kernels.DECODE_MAX_KEYS

    def graph_key(self, shape) -> bool:
        """Which of the two decode streams a step of single tokens takes (``kernels.decode_prefers_list``): a captured
        step holds the kernel that was chosen when it was captured, so even and uneven batches get graphs of their own."""
        return kernels.decode_prefers_list(shape.longest, shape.total, shape.num_requests, self.num_kv_heads)

    def work_list(self, ctx, first_request: int):
        """(tile_req, tile_tok0, tile_seg, tile_slot, places) of the general kernel on the device for the requests from
        ``first_request`` on; ``tile_seg`` and ``tile_slot`` are None without shared tiles. Made once per step and kept
        in ``ctx.memo``: every attention layer of these sizes uses the same list."""
        key = ("attention_work_list", self.tokens_per_tile, first_request, self.max_key_segments, self.num_kv_heads)
        tiles = ctx.memo.get(key)
        if tiles is None:
            req, tok0, seg, slot, places = AttentionPolicy.plan_items(ctx.starts, ctx.q_lens, self.tokens_per_tile, first_request,
                                                                      self.max_key_segments, self.num_kv_heads, kernels.sm_count())
            rows = [req, tok0] + ([seg, slot] if places else [])
            host = torch.tensor(rows, dtype=torch.int32).pin_memory()
            dev = host.to(ctx.device, non_blocking=True)
            tiles = (dev[0].contiguous(), dev[1].contiguous(), dev[2].contiguous() if places else None,
                     dev[3].contiguous() if places else None, places)
            ctx.memo[key] = tiles
        return tiles

    def attend(self, ctx, qkv: torch.Tensor, out: torch.Tensor, cache: LayerCache) -> None:
        """Causal attention of the step's query rows (the first ``num_heads * head_dim`` columns of ``qkv``) over the
        pages of ``cache``."""
        page_size = cache.pages.shape[3]
        tables = ctx.block_tables[cache.group]
        if ctx.max_q_len == 1:
            # every request brings one token: row r is request r
            kernels.decode_attention(qkv, qkv.stride(0), out, cache.pages, tables, ctx.ctx_len,
                                     ctx.decode_ctx_bound or ctx.max_ctx_len, self.num_heads, self.num_kv_heads,
                                     self.head_dim, page_size, self.window or 0, self.scale, uneven=self.graph_key(ctx.shape()))
            return
        lead = 0
        if ctx.leading_single and ctx.leading_longest >= AttentionPolicy.SPLIT_DECODE_MIN_CONTEXT:
            # Decoded tokens beside portions of prompts: as a tile of the general kernel a single token has one block
            # per key/value head walk all its keys alone, which a long context makes the longest block of the step by
            # far. The decode kernel spreads those keys over the SMs; the general kernel takes the other requests.
            lead = ctx.leading_single
            kernels.decode_attention(qkv, qkv.stride(0), out[:lead], cache.pages, tables[:lead], ctx.ctx_len[:lead],
                                     ctx.leading_longest, self.num_heads, self.num_kv_heads, self.head_dim, page_size,
                                     self.window or 0, self.scale,
                                     uneven=kernels.decode_prefers_list(ctx.leading_longest, ctx.leading_keys, lead, self.num_kv_heads))
        tile_req, tile_tok0, tile_seg, tile_slot, places = self.work_list(ctx, lead)
        kernels.paged_attention(qkv, qkv.stride(0), out, cache.pages, tables, ctx.q_start, ctx.ctx_len, tile_req, tile_tok0,
                                self.num_heads, self.num_kv_heads, self.head_dim, page_size, self.window or 0, self.scale,
                                self.tokens_per_tile, tile_seg, tile_slot, places)
