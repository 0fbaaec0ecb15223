"""What the parts see of one step: the tokens of the batch and where their requests stand.

A step holds, for each request in it, a run of consecutive new tokens (a portion of a prompt, or
one decoded token). All runs are laid end to end on one token axis of length ``num_tokens``.
"""

from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Tuple

import torch

from ..ops import kernels


class StepContext:
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
        self.decode_keys = (0, 0)            # decode steps: the most keys a request sees, and the keys of all
        self.leading_single = 0              # requests at the front of the step that bring one token each
        self.leading_longest = 0             # the most keys one of them sees
        self.leading_keys = 0                # the keys they see together
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
        self._tiles: Dict[Tuple[int, int, int, int], tuple] = {}

    def attention_tiles(self, tokens_per_tile: int, first_request: int = 0, max_segments: int = 1, num_kv_heads: int = 1):
        """(tile_req, tile_tok0, tile_seg, tile_slot, places): the work list of the general attention kernel for the
        requests from ``first_request`` on. A tile is ``tokens_per_tile`` consecutive new tokens of a request. Where
        the kernel can share a tile's keys among items (``max_segments`` > 1) and the tiles are too few to give every
        SM a block (few new tokens over long contexts), a tile comes as several consecutive items, each with an equal
        share of its keys and at least ``SPLIT_KEYS_MIN_TILES`` key tiles. ``tile_seg`` is then the
        item's place among its tile's items and their number (<< 8), ``tile_slot`` the first of the tile's ``places``
        for sums; without shared tiles both are None."""
        key = (tokens_per_tile, first_request, max_segments, num_kv_heads)
        tiles = self._tiles.get(key)
        if tiles is None:
            req, tok0, seg, slot, places = self.plan_attention_items(self.starts, self.q_lens, tokens_per_tile, first_request,
                                                                     max_segments, num_kv_heads, kernels.sm_count())
            rows = [req, tok0] + ([seg, slot] if places else [])
            host = torch.tensor(rows, dtype=torch.int32).pin_memory()
            dev = host.to(self.device, non_blocking=True)
            tiles = (dev[0].contiguous(), dev[1].contiguous(), dev[2].contiguous() if places else None,
                     dev[3].contiguous() if places else None, places)
            self._tiles[key] = tiles
        return tiles

    @classmethod
    def plan_attention_items(cls, starts: List[int], q_lens: List[int], tokens_per_tile: int, first_request: int,
                             max_segments: int, num_kv_heads: int, sms: int):
        """The work list of ``attention_tiles`` as host lists (request, first token, item of its tile | items << 8,
        first place of the tile) and the number of places, for a GPU of ``sms`` SMs."""
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

    def attention(self, mixer, qkv: torch.Tensor, out: torch.Tensor, cache) -> None:
        """Causal attention of the step's query rows (the first ``num_heads * head_dim`` columns of
        ``qkv``) over the pages of ``cache``."""
        page_size = cache.pages.shape[3]
        if self.max_q_len == 1:
            # every request brings one token: row r is request r
            kernels.decode_attention(qkv, qkv.stride(0), out, cache.pages, self.block_tables[cache.group],
                                     self.ctx_len, self.decode_ctx_bound or self.max_ctx_len, mixer.num_heads,
                                     mixer.num_kv_heads, mixer.head_dim, page_size, mixer.window or 0, mixer.scale,
                                     uneven=kernels.decode_prefers_list(*self.decode_keys, self.num_requests, mixer.num_kv_heads))
            return
        lead = 0
        if self.leading_single and self.leading_longest >= self.SPLIT_DECODE_MIN_CONTEXT:
            # Decoded tokens beside portions of prompts: as a tile of the general kernel a single token has one block
            # per key/value head walk all its keys alone, which a long context makes the longest block of the step by
            # far. The decode kernel spreads those keys over the SMs; the general kernel takes the other requests.
            lead = self.leading_single
            tables = self.block_tables[cache.group]
            kernels.decode_attention(qkv, qkv.stride(0), out[:lead], cache.pages, tables[:lead], self.ctx_len[:lead],
                                     self.leading_longest, mixer.num_heads, mixer.num_kv_heads, mixer.head_dim, page_size,
                                     mixer.window or 0, mixer.scale,
                                     uneven=kernels.decode_prefers_list(self.leading_longest, self.leading_keys, lead, mixer.num_kv_heads))
        tile_req, tile_tok0, tile_seg, tile_slot, places = self.attention_tiles(mixer.tokens_per_tile, lead, getattr(mixer, "max_key_segments", 1),
                                                                                mixer.num_kv_heads)
        kernels.paged_attention(qkv, qkv.stride(0), out, cache.pages, self.block_tables[cache.group], self.q_start,
                                self.ctx_len, tile_req, tile_tok0, mixer.num_heads, mixer.num_kv_heads,
                                mixer.head_dim, page_size, mixer.window or 0, mixer.scale, mixer.tokens_per_tile,
                                tile_seg, tile_slot, places)
