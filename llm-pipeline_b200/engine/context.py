"""What the parts see of one step: the tokens of the batch and where their requests stand.

A step holds, for each request in it, a run of consecutive new tokens (a portion of a prompt, or
one decoded token). All runs are laid end to end on one token axis of length ``num_tokens``.
"""

from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Tuple

import torch

from ..ops import kernels


class StepContext:
    def __init__(self, device: torch.device, dtype: torch.dtype):
        self.device, self.dtype = device, dtype
        self.num_tokens = 0
        self.num_requests = 0
        # host side
        self.req_ids: List[Hashable] = []
        self.starts: List[int] = []          # tokens already cached, per request
        self.q_lens: List[int] = []          # new tokens in this step, per request
        self.max_q_len = 0
        self.max_ctx_len = 0
        self.num_logit_rows = 0
        self.table_width = 0
        self.decode_ctx_bound = 0            # when set: the context length the decode kernels size their grid for
        self.contexts_uneven = False         # decode steps: one request is much longer than the average
        # device side (int32)
        self.token_ids: torch.Tensor = None  # [N]
        self.positions: torch.Tensor = None  # [N]
        self.q_start: torch.Tensor = None    # [R + 1]
        self.ctx_len: torch.Tensor = None    # [R] keys visible to the request after this step
        self.slots: torch.Tensor = None      # [R] state slot of each request
        self.token_request: torch.Tensor = None  # [N] index of the request in this step
        self.logit_rows: Optional[torch.Tensor] = None  # [M]
        self.slot_mapping: List[torch.Tensor] = []      # per cache group: [N] physical token slot (-1: none)
        self.block_tables: List[torch.Tensor] = []      # per cache group: [R, width]
        self.position_tables: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._tiles: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    def attention_tiles(self, tokens_per_tile: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(tile_req, tile_tok0): the query tiles of the general attention kernel, one tile per
        ``tokens_per_tile`` consecutive new tokens of a request."""
        tiles = self._tiles.get(tokens_per_tile)
        if tiles is None:
            # in the order of the keys they see: the kernels start the last tile first, the longest blocks lead
            found = []
            for r, n in enumerate(self.q_lens):
                before = self.starts[r]
                for t in range(0, n, tokens_per_tile):
                    found.append((before + min(t + tokens_per_tile, n), r, t))
            found.sort()
            req = [f[1] for f in found]
            tok0 = [f[2] for f in found]
            host = torch.tensor([req, tok0], dtype=torch.int32).pin_memory()
            dev = host.to(self.device, non_blocking=True)
            tiles = (dev[0].contiguous(), dev[1].contiguous())
            self._tiles[tokens_per_tile] = tiles
        return tiles

    def attention(self, mixer, qkv: torch.Tensor, out: torch.Tensor, cache) -> None:
        """Causal attention of the step's query rows (the first ``num_heads * head_dim`` columns of
        ``qkv``) over the pages of ``cache``."""
        page_size = cache.pages.shape[3]
        if self.max_q_len == 1:
            # every request brings one token: row r is request r
            kernels.decode_attention(qkv, qkv.stride(0), out, cache.pages, self.block_tables[cache.group],
                                     self.ctx_len, self.decode_ctx_bound or self.max_ctx_len, mixer.num_heads,
                                     mixer.num_kv_heads, mixer.head_dim, page_size, mixer.window or 0, mixer.scale,
                                     uneven=self.contexts_uneven or kernels.decode_rows_uneven(self.num_requests, mixer.num_kv_heads))
            return
        tile_req, tile_tok0 = self.attention_tiles(mixer.tokens_per_tile)
        kernels.paged_attention(qkv, qkv.stride(0), out, cache.pages, self.block_tables[cache.group], self.q_start,
                                self.ctx_len, tile_req, tile_tok0, mixer.num_heads, mixer.num_kv_heads,
                                mixer.head_dim, page_size, mixer.window or 0, mixer.scale, mixer.tokens_per_tile)
