"""The cache manager: paged keys/values with a block table per request, and state slots.

The reference's ``PagedAttentionManager`` keeps a free list of blocks and a list of block ids per
sequence, sized once for the prompt, and no model code ever reads its blocks
(src/llm_pipeline/inference/paged_attention.py:73-187; pages are allocated at
src/llm_pipeline/inference/qwen3_engine.py:362). When blocks run out it silently evicts other
sequences (paged_attention.py:264-286). Here the pages are what the attention kernels read and
write; they grow with the request; and the manager never evicts: ``reserve`` reports failure and
the scheduler decides.

Layers with the same need form a *group* with pages of its own: one page id addresses the same
page in every cache of the group (a tensor ``[num_pages, *spec.page_shape(page_size)]`` per cache:
``[num_pages, 2, kv_heads, page_size, head_dim]`` for keys and values). A group whose layers see only a window of keys gives pages back as soon as every token
in them has left the window; its block table then holds -1 there. Beside the pages, every live
request owns a *slot*: an index into per-cache state tensors of fixed size per request, zeroed
when the slot is handed out.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple, Union

import torch

from .spec import PagesSpec, StateSpec


class CacheError(RuntimeError):
    pass


class PagePool:
    """Page ids 0..n-1 with a LIFO free list: the pages freed last are handed out first (in the order
    in which their holder held them), so reuse happens early and deterministically. Double frees and
    foreign ids are errors."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._is_free = [True] * num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        """n pages, or None (and nothing taken) when fewer are free."""
        if n < 0:
            raise CacheError("negative page count")
        if n > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._is_free[p] = False
        self.high_water = max(self.high_water, self.num_used)
        return pages

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise CacheError(f"page {p} does not belong to this pool")
            if self._is_free[p]:
                raise CacheError(f"page {p} freed twice")
        # In reverse, so that the pages of a run come out again in the order in which they were held: a request that
        # gets the pages of one that ended holds ascending ids again, and the attention kernels bring pages whose ids
        # follow one another in one TMA box.
        for p in reversed(pages):
            self._is_free[p] = True
            self._free.append(p)

    def free_ids(self) -> List[int]:
        return list(self._free)


@dataclass
class CacheGroup:
    spec: PagesSpec
    cache_ids: List[int]
    pool: PagePool
    tables: Dict[Hashable, List[int]] = field(default_factory=dict)
    tensors: Dict[int, torch.Tensor] = field(default_factory=dict)


@dataclass
class _Request:
    slot: int
    length: int = 0
    admission: int = 0       # counts admissions of the manager: tells a request from an earlier one of the same name


class CacheManager:
    """``cache_specs[i]`` is what cache id ``i`` needs: ``(PagesSpec | None, StateSpec | None)``.
    ``num_pages`` is the page count of every group, or a list with one count per group (groups
    are numbered in order of first appearance). With ``device=None`` no tensor is allocated and
    the manager only keeps books (used by the scheduler's tests)."""

    def __init__(self, cache_specs: Sequence[Tuple[Optional[PagesSpec], Optional[StateSpec]]], page_size: int,
                 num_pages: Union[int, Sequence[int]], max_requests: int, max_request_tokens: int,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16):
        if page_size <= 0:
            raise CacheError(f"page size must be positive, got {page_size}")
        if max_requests <= 0:
            raise CacheError("max_requests must be positive")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_request_tokens = int(max_request_tokens)
        self.table_width = max(1, -(-self.max_request_tokens // self.page_size))
        self.device, self.dtype = device, dtype
        self.groups: List[CacheGroup] = []
        self.group_of_cache: Dict[int, int] = {}
        keys: Dict[tuple, int] = {}
        for cache_id, (kv, _state) in enumerate(cache_specs):
            if kv is None:
                continue
            key = kv.group_key()
            if key not in keys:
                keys[key] = len(self.groups)
                count = num_pages if isinstance(num_pages, int) else num_pages[len(self.groups)]
                self.groups.append(CacheGroup(kv, [], PagePool(int(count))))
            self.groups[keys[key]].cache_ids.append(cache_id)
            self.group_of_cache[cache_id] = keys[key]
        self.state_specs: Dict[int, StateSpec] = {i: s for i, (_kv, s) in enumerate(cache_specs) if s is not None}
        self.states: Dict[int, torch.Tensor] = {}
        if device is not None:
            for group in self.groups:
                shape = (group.pool.num_pages,) + tuple(group.spec.page_shape(self.page_size))
                for cache_id in group.cache_ids:
                    group.tensors[cache_id] = torch.zeros(shape, dtype=group.spec.dtype or dtype, device=device)
            for cache_id, spec in self.state_specs.items():
                self.states[cache_id] = torch.zeros((self.max_requests,) + tuple(spec.shape), dtype=spec.dtype,
                                                    device=device)
        self._free_slots: List[int] = list(range(self.max_requests - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}
        self._admissions = 0
        self.pages_reused = 0
        self._ever_used = [set() for _ in self.groups]

    # -- requests and slots ----------------------------------------------------------------
    def __contains__(self, req_id: Hashable) -> bool:
        return req_id in self._requests

    @property
    def num_live(self) -> int:
        return len(self._requests)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, req_id: Hashable) -> int:
        """Give the request a slot (its state zeroed) and empty block tables."""
        if req_id in self._requests:
            raise CacheError(f"request {req_id!r} is already live")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        self._admissions += 1
        self._requests[req_id] = _Request(slot, admission=self._admissions)
        for group in self.groups:
            group.tables[req_id] = []
        for tensor in self.states.values():
            tensor[slot].zero_()
        return slot

    def slot_of(self, req_id: Hashable) -> int:
        return self._requests[req_id].slot

    def admission(self, req_id: Hashable) -> int:
        """A number that no other admission of this manager has: a request that ended (or was preempted) and came
        back under the same name has another one, and block tables remembered for the old one are void."""
        return self._requests[req_id].admission

    def length(self, req_id: Hashable) -> int:
        """Tokens of the request whose keys/values (or state) the cache holds."""
        return self._requests[req_id].length

    def block_table(self, req_id: Hashable, group: int) -> List[int]:
        return self.groups[group].tables[req_id]

    # -- pages -----------------------------------------------------------------------------
    def _first_needed_page(self, group: CacheGroup, start: int) -> int:
        """First logical page a step that starts at token ``start`` still has to hold."""
        if group.spec.window is None:
            return 0
        lowest_key = max(0, start - group.spec.window + 1)
        return lowest_key // self.page_size

    def pages_short(self, req_id: Hashable, new_length: int) -> List[int]:
        """Per group, how many pages ``reserve(req_id, new_length)`` would have to take."""
        out = []
        for group in self.groups:
            table = group.tables.get(req_id, ())   # a request that is not admitted yet holds nothing
            want = -(-new_length // self.page_size)
            out.append(max(0, want - len(table)))
        return out

    def can_reserve(self, req_id: Hashable, new_length: int, spare: Optional[List[int]] = None,
                    short: Optional[List[int]] = None) -> bool:
        """True when every group has the pages; ``spare`` (one count per group) is subtracted from
        the free pages first, for callers that plan several reservations before making them.
        ``short``: the result of ``pages_short`` for the same arguments, when the caller has it."""
        if new_length > self.max_request_tokens:
            return False
        if short is None:
            short = self.pages_short(req_id, new_length)
        for g, group in enumerate(self.groups):
            if short[g] > group.pool.num_free - (spare[g] if spare else 0):
                return False
        return True

    def reserve(self, req_id: Hashable, new_length: int) -> bool:
        """Make sure pages exist for tokens < new_length in every group; all or nothing."""
        if req_id not in self._requests:
            raise CacheError(f"request {req_id!r} is not live")
        if new_length > self.max_request_tokens:
            raise CacheError(f"request {req_id!r} would hold {new_length} tokens, the limit is {self.max_request_tokens}")
        short = self.pages_short(req_id, new_length)
        if not any(short):
            return True                                   # the pages it holds cover the new length
        if not self.can_reserve(req_id, new_length, None, short):
            return False
        for g, group in enumerate(self.groups):
            pages = group.pool.alloc(short[g])
            assert pages is not None
            for p in pages:
                if p in self._ever_used[g]:
                    self.pages_reused += 1
                self._ever_used[g].add(p)
            group.tables[req_id].extend(pages)
        return True

    def commit(self, req_id: Hashable, new_length: int) -> None:
        """The step that wrote tokens up to new_length has been issued: record the length and
        give back the pages that no later token of this request can see."""
        request = self._requests[req_id]
        if new_length < request.length:
            raise CacheError("a request's length cannot shrink")
        request.length = new_length
        for group in self.groups:
            if group.spec.window is None:
                continue
            table = group.tables[req_id]
            keep_from = self._first_needed_page(group, new_length)
            gone = [p for p in table[:keep_from] if p >= 0]
            if gone:
                group.pool.free(gone)
                for i in range(min(keep_from, len(table))):
                    table[i] = -1

    def free(self, req_id: Hashable) -> None:
        """The request ended (or was preempted): all its pages and its slot go back."""
        request = self._requests.pop(req_id, None)
        if request is None:
            raise CacheError(f"request {req_id!r} is not live (freed twice?)")
        for group in self.groups:
            table = group.tables.pop(req_id)
            group.pool.free([p for p in table if p >= 0])
        self._free_slots.append(request.slot)

    # -- views for the step function -------------------------------------------------------
    def pages_tensor(self, cache_id: int) -> torch.Tensor:
        return self.groups[self.group_of_cache[cache_id]].tensors[cache_id]

    def state_tensor(self, cache_id: int) -> Optional[torch.Tensor]:
        return self.states.get(cache_id)

    def token_slot(self, req_id: Hashable, group: int, position: int) -> int:
        """Physical token slot (page * page_size + offset) of a position, or -1 without a page."""
        page = self.groups[group].tables[req_id][position // self.page_size]
        return -1 if page < 0 else page * self.page_size + position % self.page_size

    @staticmethod
    def bytes_per_page(cache_specs, page_size: int, dtype: torch.dtype) -> List[int]:
        """Per group (in the order the manager numbers them), the bytes one page id costs over all caches of the
        group: what a memory budget divides by."""
        keys: Dict[tuple, int] = {}
        out: List[int] = []
        for pages, _state in cache_specs:
            if pages is None:
                continue
            key = pages.group_key()
            if key not in keys:
                keys[key] = len(out)
                out.append(0)
            out[keys[key]] += pages.bytes_per_token(dtype) * page_size
        return out

    # -- bookkeeping -----------------------------------------------------------------------
    def stats(self) -> Dict[str, object]:
        return {
            "live_requests": len(self._requests),
            "free_slots": len(self._free_slots),
            "pages_free": [g.pool.num_free for g in self.groups],
            "pages_used": [g.pool.num_used for g in self.groups],
            "pages_high_water": [g.pool.high_water for g in self.groups],
            "pages_reused": self.pages_reused,
        }

    def check(self) -> None:
        """Every page is either free or in exactly one block table; every slot likewise."""
        for g, group in enumerate(self.groups):
            seen = {}
            for req_id, table in group.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheError(f"group {g}: page {p} held by {seen[p]!r} and {req_id!r}")
                    seen[p] = req_id
            free = group.pool.free_ids()
            if len(set(free)) != len(free):
                raise CacheError(f"group {g}: a page is twice in the free list")
            if set(free) & set(seen):
                raise CacheError(f"group {g}: a page is both free and held")
            if len(free) + len(seen) != group.pool.num_pages:
                raise CacheError(f"group {g}: {group.pool.num_pages - len(free) - len(seen)} pages lost")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots) or \
                len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("slot bookkeeping is inconsistent")
