"""What a mixer asks of the cache manager.

``KVPagesSpec``: keys and values of every token in pages; ``window`` (None = all keys) tells the
manager that pages whose tokens have all left the window may be given back while the request
lives. ``StateSpec``: a tensor of fixed size per request (recurrent state, running statistics);
it lives in the request's slot and is zeroed when the slot is handed out.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVPagesSpec:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self):
        return ("kv", self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
