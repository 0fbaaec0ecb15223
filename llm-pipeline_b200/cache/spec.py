"""What a mixer asks of the cache manager.

``PagesSpec``: something per token, kept in pages. The spec says what one page looks like
(``page_shape(page_size)``: the tensor of a cache is ``[num_pages, *page_shape]``), optionally its
element type (default: the cache's), and ``window`` (None = every earlier token): pages whose
tokens have all left the window may be given back while the request lives. Caches whose specs have
the same ``group_key()`` share page ids and block tables. The manager, the memory budget and the
benchmark read sizes from the spec alone (``elements_per_token``, ``bytes_per_token``).

* ``KVPagesSpec``: keys and values of attention, page ``[2, kv_heads, page_size, head_dim]``.
* ``TokenPagesSpec``: any payload of a fixed shape per token, page ``[page_size, *token_shape]``
  (a latent vector, keys and values of different widths packed side by side, ...).

``StateSpec``: a tensor of fixed size per request (recurrent state, running statistics); it lives
in the request's slot and is zeroed when the slot is handed out.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


class PagesSpec:
    """Base of the paged specs; a subclass is a frozen dataclass with a ``window`` field."""

    window: Optional[int] = None
    dtype: Optional[torch.dtype] = None          # None: the element type the cache was made with

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        raise NotImplementedError

    def group_key(self):
        """Caches with equal keys form one group: one pool of page ids, one block table per request."""
        return (type(self).__name__, self.page_shape(1), self.dtype, self.window)

    def elements_per_token(self) -> int:
        count = 1
        for n in self.page_shape(1):
            count *= n
        return count

    def bytes_per_token(self, cache_dtype: torch.dtype) -> int:
        return self.elements_per_token() * torch.empty((), dtype=self.dtype or cache_dtype).element_size()


@dataclass(frozen=True)
class KVPagesSpec(PagesSpec):
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (2, self.num_kv_heads, page_size, self.head_dim)

    def group_key(self):
        return ("kv", self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class TokenPagesSpec(PagesSpec):
    token_shape: Tuple[int, ...]
    window: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (page_size,) + tuple(self.token_shape)


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
