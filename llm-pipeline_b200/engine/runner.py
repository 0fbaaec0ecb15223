"""The step function: run a batch of (request, its next tokens) from the cache and return the
logits at the wanted places.

The nearest thing in the reference is one call of
``model(input_ids, attention_mask, past_key_values, use_cache)``
(src/llm_pipeline/models/qwen3/custom_builder.py:393-421), which takes a dense rectangle of
tokens, returns logits for every position and a cache tuple re-built by concatenation. Here a
step takes any mix of prompt portions and single decoded tokens, runs only those tokens against
the paged cache that earlier steps left, and computes the output head for the wanted rows only.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import torch

from ..cache import CacheManager
from ..models.model import Model
from ..parts import LayerCache
from .context import StepContext


class OutOfPages(RuntimeError):
    """The step's tokens do not fit the page pool."""


@dataclass
class StepEntry:
    """The next ``tokens`` of request ``req_id``; ``want`` lists the places among these tokens
    (0-based) whose logits are asked for."""

    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class _CacheViews:
    def __init__(self, cache: CacheManager):
        self.cache = cache

    def view(self, cache_id: int, writes: bool) -> LayerCache:
        group = self.cache.group_of_cache.get(cache_id)
        pages = self.cache.pages_tensor(cache_id) if group is not None else None
        return LayerCache(pages=pages, group=group, state=self.cache.state_tensor(cache_id), writes=writes)


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager):
        if model.device is None:
            raise RuntimeError("the model has no weights yet: call model.load() first")
        if model.device.type != "cuda":
            raise RuntimeError(f"the engine runs on CUDA devices only, the model is on {model.device}")
        self.model, self.cache = model, cache
        self.device, self.dtype = model.device, model.dtype
        self.vocab_size = model.spec.vocab_size
        self._views = _CacheViews(cache)
        self.steps = 0
        self.tokens_run = 0
        self.last_h2d_bytes = 0

    # -- building the step's index arrays ------------------------------------------------------
    def _prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        cache = self.cache
        ctx = StepContext(self.device, self.dtype)
        seen = set()
        spare = [0] * len(cache.groups)
        admitted = []
        try:
            for e in entries:
                if e.req_id in seen:
                    raise ValueError(f"request {e.req_id!r} appears twice in one step")
                seen.add(e.req_id)
                n = len(e.tokens)
                if n == 0:
                    raise ValueError(f"request {e.req_id!r} brings no tokens")
                for t in e.tokens:
                    if not 0 <= int(t) < self.vocab_size:
                        raise ValueError(f"token id {t} of request {e.req_id!r} is outside the vocabulary "
                                         f"of {self.vocab_size}")
                for w in e.want:
                    if not 0 <= int(w) < n:
                        raise ValueError(f"request {e.req_id!r} wants logits at place {w} of {n} tokens")
                if e.req_id not in cache:
                    cache.admit(e.req_id)
                    admitted.append(e.req_id)
                start = cache.length(e.req_id)
                if start + n > cache.max_request_tokens:
                    raise OutOfPages(f"request {e.req_id!r} would hold {start + n} tokens; the cache was made for "
                                     f"{cache.max_request_tokens} per request")
                if not cache.can_reserve(e.req_id, start + n, spare):
                    raise OutOfPages(f"no pages left for {n} more tokens of request {e.req_id!r} "
                                     f"(free pages per group: {[g.pool.num_free for g in cache.groups]})")
                short = cache.pages_short(e.req_id, start + n)
                spare = [a + b for a, b in zip(spare, short)]
        except Exception:
            for req_id in admitted:
                cache.free(req_id)
            raise
        for e in entries:
            ok = cache.reserve(e.req_id, cache.length(e.req_id) + len(e.tokens))
            assert ok

        R = len(entries)
        N = sum(len(e.tokens) for e in entries)
        ps = cache.page_size
        token_ids: List[int] = []
        positions: List[int] = []
        token_request: List[int] = []
        q_start = [0]
        ctx_len, slots, rows = [], [], []
        for r, e in enumerate(entries):
            start, n = cache.length(e.req_id), len(e.tokens)
            ctx.req_ids.append(e.req_id)
            ctx.starts.append(start)
            ctx.q_lens.append(n)
            token_ids.extend(int(t) for t in e.tokens)
            positions.extend(range(start, start + n))
            token_request.extend([r] * n)
            rows.extend(q_start[-1] + int(w) for w in e.want)
            q_start.append(q_start[-1] + n)
            ctx_len.append(start + n)
            slots.append(cache.slot_of(e.req_id))
        ctx.num_tokens, ctx.num_requests = N, R
        ctx.max_q_len = max(ctx.q_lens)
        ctx.max_ctx_len = max(ctx_len)
        width = max(1, -(-ctx.max_ctx_len // ps))
        flat: List[int] = token_ids + positions + token_request + q_start + ctx_len + slots + rows
        for g in range(len(cache.groups)):
            mapping: List[int] = []
            tables: List[int] = []
            for r, e in enumerate(entries):
                table = cache.block_table(e.req_id, g)
                start, n = ctx.starts[r], ctx.q_lens[r]
                for pos in range(start, start + n):
                    page = table[pos // ps]
                    mapping.append(-1 if page < 0 else page * ps + pos % ps)
                tables.extend(table[:width] + [-1] * (width - len(table[:width])))
            flat += mapping + tables
        host = torch.tensor(flat, dtype=torch.int32).pin_memory()
        dev = host.to(self.device, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4
        cursor = 0

        def take(count: int) -> torch.Tensor:
            nonlocal cursor
            out = dev[cursor:cursor + count]
            cursor += count
            return out

        ctx.token_ids, ctx.positions, ctx.token_request = take(N), take(N), take(N)
        ctx.q_start, ctx.ctx_len, ctx.slots = take(R + 1), take(R), take(R)
        ctx.logit_rows = take(len(rows)) if rows else None
        for g in range(len(cache.groups)):
            ctx.slot_mapping.append(take(N))
            ctx.block_tables.append(take(R * width).view(R, width))
        return ctx

    # -- the step ----------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries as one batch. Returns float32 logits ``[wanted, vocab]`` in the order of
        the entries and of their ``want`` lists, or None when nothing is wanted."""
        entries = list(entries)
        if not entries:
            return None
        ctx = self._prepare(entries)
        with torch.cuda.device(self.device):
            stream = self.model.forward(ctx, self._views)
            logits = self.model.logits(ctx, stream, ctx.logit_rows) if ctx.logit_rows is not None else None
        for r, e in enumerate(entries):
            self.cache.commit(e.req_id, ctx.starts[r] + ctx.q_lens[r])
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        return logits

    def release(self, req_id: Hashable) -> None:
        """The request is finished: its pages and slot go back to the pool."""
        if req_id in self.cache:
            self.cache.free(req_id)
