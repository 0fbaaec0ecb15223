"""What the parts see of one step: the tokens of the batch and where their requests stand.

A step holds, for each request in it, a run of consecutive new tokens (a portion of a prompt, or
one decoded token). All runs are laid end to end on one token axis of length ``num_tokens``.
The context states facts of the step only; what a part makes of them (which kernel an attention
mixer takes for this shape, its work lists) belongs to the part, which may keep per-step results
in ``memo`` so that its other layers find them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Hashable, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class StepShape:
    """What is known of a step of single tokens before its context exists: enough for a mixer to say which of its
    kernels such a step takes (``Mixer.graph_key``), which is part of the key of a captured decode graph."""

    num_requests: int
    longest: int          # the most keys a request sees after this step
    total: int            # the keys all requests see together


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
        self.max_ctx_len = 0                 # the most keys a request sees after this step
        self.total_ctx = 0                   # the keys all requests see together
        self.num_logit_rows = 0
        self.table_width = 0
        self.decode_ctx_bound = 0            # when set (captured steps): the context length kernels size their grids for
        self.leading_single = 0              # requests at the front of a mixed step that bring one token each
        self.leading_longest = 0             # the most keys one of them sees
        self.leading_keys = 0                # the keys they see together
        # device side (int32)
        self.token_ids: torch.Tensor = None  # [N]
        self.positions: torch.Tensor = None  # [N]: each token's place in its request (where its keys go in the cache)
        self.position_ids: torch.Tensor = None  # [streams, N]: what position encodings read; one stream: the places
        self.q_start: torch.Tensor = None    # [R + 1]
        self.ctx_len: torch.Tensor = None    # [R] keys visible to the request after this step
        self.slots: torch.Tensor = None      # [R] state slot of each request
        self.token_request: torch.Tensor = None  # [N] index of the request in this step
        self.logit_rows: Optional[torch.Tensor] = None  # [M]
        self.slot_mapping: List[torch.Tensor] = []      # per cache group: [N] physical token slot (-1: none)
        self.block_tables: List[torch.Tensor] = []      # per cache group: [R, width]
        self.position_tables: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.memo: Dict[Hashable, Any] = {}  # per-step results of parts (work lists), shared by their layers

    def shape(self) -> StepShape:
        return StepShape(self.num_requests, self.max_ctx_len, self.total_ctx)
