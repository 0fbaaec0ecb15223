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

import copy
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..models.model import Model
from ..ops import kernels, timing
from ..parts import LayerCache, ResidualStream
from .context import StepContext, StepShape


class OutOfPages(RuntimeError):
    """The step's tokens do not fit the page pool."""


@dataclass
class StepEntry:
    """The next ``tokens`` of request ``req_id``; ``want`` lists the places among these tokens
    (0-based) whose logits are asked for. ``positions``: for a model whose position encoding reads more than one
    stream of positions (``PositionEncoding.streams``), the position ids of these tokens, one sequence per stream;
    None: every stream holds the tokens' places in the request, which is what a one-stream encoding always reads."""

    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)
    positions: Optional[Sequence[Sequence[int]]] = None
    # For an entry of one token whose id is still on the device (sampled by the step before, not read back yet):
    # (int32 tensor of sampled ids, index into it). ``tokens`` then holds any valid id as a stand-in; the step copies
    # the real one into its token array on the device before it runs.
    device_token: Optional[tuple] = None


class _CacheViews:
    def __init__(self, cache: CacheManager):
        self.cache = cache

    def view(self, cache_id: int, writes: bool) -> LayerCache:
        group = self.cache.group_of_cache.get(cache_id)
        pages = self.cache.pages_tensor(cache_id) if group is not None else None
        return LayerCache(pages=pages, group=group, state=self.cache.state_tensor(cache_id), writes=writes)


class _DecodeGraph:
    """A captured decode step for one shape: its static index buffers, context, graph and output."""

    def __init__(self):
        self.seen = 0
        self.graph = None
        self.host = None
        self.dev = None
        self.ctx = None
        self.logits = None
        self.copied = None
        self.launches = 0
        self.host_np = None          # the pinned buffer as a numpy array (same memory)
        self.req_ids = None          # the requests of the last step in row order, each with its admission number
        self.table_lens = None       # per cache group and row: pages of the block table already in the buffer
        self.pieces = None           # a model that is captured in pieces: [_Piece] in the order of the schedule


class _Piece:
    """A run of scheduled layers of a captured decode step: either a CUDA graph (``graph``; it reads the float32
    residual ``inlet`` unless it is the first piece, and leaves ``outlet``: the residual after its layers, or the
    logits if it is the last piece) or layers that run eagerly every step (``graph`` None)."""

    def __init__(self, first: int, end: int):
        self.first, self.end = first, end
        self.graph = None
        self.inlet = None
        self.outlet = None


class ModelRunner:
    """``use_graphs``: steps in which every request brings exactly one token are captured in CUDA
    graphs, one per (number of requests, wanted rows, block-table width rounded up to
    ``GRAPH_WIDTH_STEP`` pages), and replayed; the first step of a shape runs eagerly. Layers with
    a part that does not declare ``graph_safe`` (a mixer that updates per-request state, a
    feed-forward whose launches depend on the data) run eagerly every step, between graphs of the runs of layers
    before and after them (``Model.pieces``); a model without a capturable layer runs eagerly as a whole. The logits
    a replayed step returns live in the graph's static buffer and are valid until the next step of the same shape."""

    GRAPH_WIDTH_STEP = 32
    CONTEXT_BOUND_STEP = 128
    MAX_GRAPHS = 64

    def __init__(self, model: Model, cache: CacheManager, use_graphs: bool = True):
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
        self._pieces = model.pieces() if hasattr(model, "pieces") else []
        # LLMP_B200_KERNEL_TIMES=1: CUDA events around every launch of every step, which then runs eagerly
        self.kernel_times = timing.KernelTimes() if timing.TIME_KERNELS else None
        use_graphs = use_graphs and self.kernel_times is None
        self.use_graphs = bool(use_graphs and any(capturable for _first, _end, capturable in self._pieces))
        self._graphs: Dict[tuple, _DecodeGraph] = {}
        self._staging: list = []             # pinned buffers for the index arrays of eager steps: (tensor, numpy view, event)
        self.graph_replays = 0
        self._context_limit = model.captured_context_limit() if hasattr(model, "captured_context_limit") else None
        self.position_streams = int(getattr(model, "position_streams", 1))
        self._token_index: Dict[tuple, tuple] = {}     # index tensors of _device_tokens, by (rows, sources)

    # -- pages for the step's tokens -----------------------------------------------------------
    def _reserve(self, entries: Sequence[StepEntry]) -> None:
        """Check the entries, admit new requests and take the pages their tokens need; all or nothing."""
        cache = self.cache
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
                if n > 16:
                    ids = np.asarray(e.tokens)
                    bad = (ids < 0) | (ids >= self.vocab_size)
                    outside = [int(ids[int(bad.argmax())])] if bad.any() else []
                else:
                    outside = [t for t in e.tokens if not 0 <= int(t) < self.vocab_size]
                if outside:
                    raise ValueError(f"token id {outside[0]} of request {e.req_id!r} is outside the vocabulary "
                                     f"of {self.vocab_size}")
                for w in e.want:
                    if not 0 <= int(w) < n:
                        raise ValueError(f"request {e.req_id!r} wants logits at place {w} of {n} tokens")
                if e.device_token is not None and n != 1:
                    raise ValueError(f"request {e.req_id!r}: only a single token can still be on the device")
                if e.positions is not None and (len(e.positions) != self.position_streams or
                                                any(len(row) != n for row in e.positions)):
                    raise ValueError(f"request {e.req_id!r} brings position ids of another shape than "
                                     f"[{self.position_streams}][{n}], one row for each stream of the model's position encoding")
                if e.req_id not in cache:
                    cache.admit(e.req_id)
                    admitted.append(e.req_id)
                start = cache.length(e.req_id)
                if start + n > cache.max_request_tokens:
                    raise OutOfPages(f"request {e.req_id!r} would hold {start + n} tokens; the cache was made for "
                                     f"{cache.max_request_tokens} per request")
                short = cache.pages_short(e.req_id, start + n)
                if not cache.can_reserve(e.req_id, start + n, spare, short):
                    raise OutOfPages(f"no pages left for {n} more tokens of request {e.req_id!r} "
                                     f"(free pages per group: {[g.pool.num_free for g in cache.groups]})")
                if any(short):
                    spare = [a + b for a, b in zip(spare, short)]
        except Exception:
            for req_id in admitted:
                cache.free(req_id)
            raise
        for e in entries:
            ok = cache.reserve(e.req_id, cache.length(e.req_id) + len(e.tokens))
            assert ok

    # -- the step's index arrays ---------------------------------------------------------------
    def _fill(self, ctx: StepContext, entries: Sequence[StepEntry], width: Optional[int] = None) -> np.ndarray:
        """Host side of the context, and the flat int32 image of its device arrays:
        token ids, positions, request of each token, q_start, ctx_len, slots, logit rows, then per
        cache group the slot mapping and the block tables (``width`` entries per request), and at the end, for a
        model with several streams of positions, the position ids stream by stream. Long runs of
        tokens (prompt portions) are filled as arrays, single tokens as scalars."""
        cache = self.cache
        ps = cache.page_size
        R = len(entries)
        starts = [cache.length(e.req_id) for e in entries]
        q_lens = [len(e.tokens) for e in entries]
        ctx_len = [s + n for s, n in zip(starts, q_lens)]
        ctx.req_ids, ctx.starts, ctx.q_lens = [e.req_id for e in entries], starts, q_lens
        first = [0] * (R + 1)
        for r, n in enumerate(q_lens):
            first[r + 1] = first[r] + n
        N = first[R]
        rows = [first[r] + int(w) for r, e in enumerate(entries) for w in e.want]
        ctx.num_tokens, ctx.num_requests = N, R
        ctx.max_q_len = max(q_lens)
        ctx.max_ctx_len = max(ctx_len)
        ctx.total_ctx = sum(ctx_len)
        lead = 0
        while lead < R and q_lens[lead] == 1:
            lead += 1
        ctx.leading_single = lead if lead < R else 0                     # a step of single tokens only is a decode step
        if ctx.leading_single:
            ctx.leading_longest, ctx.leading_keys = max(ctx_len[:lead]), sum(ctx_len[:lead])
        ctx.num_logit_rows = len(rows)
        if width is None:
            width = max(1, -(-ctx.max_ctx_len // ps))
        ctx.table_width = width
        groups = len(cache.groups)
        head = 3 * N + (R + 1) + 2 * R + len(rows)
        streams = self.position_streams if self.position_streams > 1 else 0
        flat = np.empty(head + groups * (N + R * width) + streams * N, dtype=np.int32)
        token_ids, positions, token_request = flat[0:N], flat[N:2 * N], flat[2 * N:3 * N]
        for r, e in enumerate(entries):
            at, n, start = first[r], q_lens[r], starts[r]
            if n == 1:
                token_ids[at], positions[at], token_request[at] = e.tokens[0], start, r
            else:
                token_ids[at:at + n] = e.tokens
                positions[at:at + n] = np.arange(start, start + n, dtype=np.int32)
                token_request[at:at + n] = r
        cursor = 3 * N
        flat[cursor:cursor + R + 1] = first
        cursor += R + 1
        flat[cursor:cursor + R] = ctx_len
        cursor += R
        flat[cursor:cursor + R] = [cache.slot_of(e.req_id) for e in entries]
        cursor += R
        flat[cursor:cursor + len(rows)] = rows
        cursor += len(rows)
        for g in range(groups):
            mapping = flat[cursor:cursor + N]
            tables = flat[cursor + N:cursor + N + R * width].reshape(R, width)
            tables.fill(-1)
            for r, e in enumerate(entries):
                table = cache.block_table(e.req_id, g)
                at, n, start = first[r], q_lens[r], starts[r]
                if n == 1:
                    page = table[start // ps]
                    mapping[at] = -1 if page < 0 else page * ps + start % ps
                else:
                    pos = positions[at:at + n]
                    page = np.asarray(table, dtype=np.int32)[pos // ps]
                    mapping[at:at + n] = np.where(page < 0, -1, page * ps + pos % ps)
                k = min(width, len(table))
                tables[r, :k] = table[:k]
            cursor += N + R * width
        if streams:
            ids = flat[cursor:cursor + streams * N].reshape(streams, N)
            for r, e in enumerate(entries):
                at, n = first[r], q_lens[r]
                ids[:, at:at + n] = positions[at:at + n] if e.positions is None else np.asarray(e.positions, dtype=np.int32)
        return flat

    def _to_device(self, flat: np.ndarray) -> torch.Tensor:
        """The step's index arrays on the device: through one of a few pinned staging buffers that are reused once
        the copy out of them has completed (no pinned allocation per step), one asynchronous copy."""
        n = flat.size
        chosen = None
        for buffer in self._staging:
            if buffer[0].numel() >= n and buffer[2].query():
                chosen = buffer
                break
        if chosen is None:
            if len(self._staging) >= 4:
                self._staging.pop(0)
            host = torch.empty(max(4096, 2 * n), dtype=torch.int32).pin_memory()
            chosen = (host, host.numpy(), torch.cuda.Event())
            self._staging.append(chosen)
        host, view, copied = chosen
        view[:n] = flat
        dev = torch.empty(n, dtype=torch.int32, device=self.device)
        dev.copy_(host[:n], non_blocking=True)
        copied.record()
        self.last_h2d_bytes = n * 4
        return dev

    def _device_tokens(self, token_ids: torch.Tensor, entries: Sequence[StepEntry], first_rows: Sequence[int]) -> None:
        """Copy the ids that are still on the device (``StepEntry.device_token``) into the step's token array, on the
        stream, after the array's copy from the host and before the model runs."""
        rows = [(first_rows[r], e.device_token) for r, e in enumerate(entries) if e.device_token is not None]
        if not rows:
            return
        source = rows[0][1][0]
        if (len(rows) == source.numel() and all(src is source for _row, (src, _i) in rows) and
                all(row == rows[0][0] + k and i == k for k, (row, (_src, i)) in enumerate(rows))):
            token_ids[rows[0][0]:rows[0][0] + len(rows)].copy_(source)        # the usual case: the same requests go on
            return
        for src in {id(t): t for _row, (t, _i) in rows}.values():
            mine = [(row, i) for row, (t, i) in rows if t is src]
            key = (id(src.device), tuple(mine))
            index = self._token_index.get(key)
            if index is None:
                if len(self._token_index) > 256:
                    self._token_index.clear()
                index = self._token_index[key] = (torch.tensor([row for row, _ in mine], dtype=torch.long, device=self.device),
                                                  torch.tensor([i for _, i in mine], dtype=torch.long, device=self.device))
            token_ids.index_copy_(0, index[0], src.index_select(0, index[1]))

    def _bind(self, ctx: StepContext, dev: torch.Tensor) -> None:
        """Point the context's device arrays at their places in the flat buffer."""
        N, R, width = ctx.num_tokens, ctx.num_requests, ctx.table_width
        cursor = 0

        def take(count: int) -> torch.Tensor:
            nonlocal cursor
            out = dev[cursor:cursor + count]
            cursor += count
            return out

        ctx.token_ids, ctx.positions, ctx.token_request = take(N), take(N), take(N)
        ctx.q_start, ctx.ctx_len, ctx.slots = take(R + 1), take(R), take(R)
        ctx.logit_rows = take(ctx.num_logit_rows) if ctx.num_logit_rows else None
        ctx.slot_mapping, ctx.block_tables = [], []
        for _g in range(len(self.cache.groups)):
            ctx.slot_mapping.append(take(N))
            ctx.block_tables.append(take(R * width).view(R, width))
        streams = self.position_streams
        ctx.position_ids = take(streams * N).view(streams, N) if streams > 1 else ctx.positions.view(1, N)

    @classmethod
    def decode_graph_shape(cls, longest: int, page_size: int, max_request_tokens: int, limit: Optional[int] = None):
        """(block-table width, context bound) of the graph that serves a decode step whose longest request sees
        ``longest`` keys. The width is the request's pages rounded up to ``GRAPH_WIDTH_STEP``; the bound, for which the
        captured kernels size their grids and scratch, is what that width can hold but never more than a request
        may grow to (rounded up to ``CONTEXT_BOUND_STEP``). None as bound: it is beyond ``limit``, the longest context
        the model's mixers take in a captured step (``Mixer.captured_context_limit``), so the step must run eagerly
        with its real length."""
        step_w = cls.GRAPH_WIDTH_STEP
        width = -(-max(1, -(-longest // page_size)) // step_w) * step_w
        split = cls.CONTEXT_BOUND_STEP
        bound = min(width * page_size, -(-max(max_request_tokens, longest) // split) * split)
        return width, (bound if limit is None or bound <= limit else None)

    def _prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserve pages and build the step context with its arrays on the device (one copy)."""
        self._reserve(entries)
        return self._prepare_reserved(entries)

    def _prepare_reserved(self, entries: Sequence[StepEntry]) -> StepContext:
        ctx = StepContext(self.device, self.dtype)
        self._bind(ctx, self._to_device(self._fill(ctx, entries)))
        if any(e.device_token is not None for e in entries):
            first, at = [], 0
            for e in entries:
                first.append(at)
                at += len(e.tokens)
            self._device_tokens(ctx.token_ids, entries, first)
        return ctx

    def _run(self, ctx: StepContext) -> Optional[torch.Tensor]:
        stream = self.model.forward(ctx, self._views)
        return self.model.logits(ctx, stream, ctx.logit_rows) if ctx.logit_rows is not None else None

    # -- captured decode steps -------------------------------------------------------------------
    def _decode_graph_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        cache = self.cache
        self._reserve(entries)
        ps = cache.page_size
        lengths = [cache.length(e.req_id) + 1 for e in entries]
        longest = max(lengths)
        width, bound = self.decode_graph_shape(longest, ps, cache.max_request_tokens, self._context_limit)
        if bound is None:
            # the width bucket reaches past what the decode kernels take although the request does not: no graph
            ctx = self._prepare_reserved(entries)
            return self._finish(ctx, entries, self._run(ctx))
        # a graph holds the kernels that were chosen when it was captured; where a mixer's choice follows the step's
        # shape (even and uneven contexts in attention), the mixers say so and such steps get graphs of their own
        which = self.model.graph_key(StepShape(len(entries), longest, sum(lengths)))
        key = (len(entries), tuple(len(e.want) for e in entries), width, which)
        slot = self._graphs.get(key)
        if slot is None:
            if len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            slot = self._graphs[key] = _DecodeGraph()
        slot.seen += 1
        if slot.seen == 1:
            # first step of this shape: run eagerly (this also lets libraries set themselves up)
            ctx = self._prepare_reserved(entries)
            return self._finish(ctx, entries, self._run(ctx))
        if slot.graph is None:
            slot.ctx = StepContext(self.device, self.dtype)
            flat = self._fill(slot.ctx, entries, width)
            slot.host = torch.from_numpy(flat).pin_memory()
            slot.host_np = slot.host.numpy()
            self._remember(slot, entries)
            slot.dev = slot.host.to(self.device)
            self._bind(slot.ctx, slot.dev)
            slot.ctx.decode_ctx_bound = bound
            slot.copied = torch.cuda.Event()
            torch.cuda.synchronize(self.device)
            before = kernels.launch_count
            if len(self._pieces) == 1:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    slot.logits = self._run(slot.ctx)
                slot.graph = graph
            else:
                self._capture_pieces(slot)
            slot.launches = kernels.launch_count - before
            kernels.launch_count = before
        else:
            slot.copied.synchronize()            # the previous copy out of the pinned buffer is done
            if slot.req_ids == [(e.req_id, cache.admission(e.req_id)) for e in entries]:
                self._refill(slot, entries, width)
            else:
                flat = self._fill(slot.ctx, entries, width)
                slot.host_np[:flat.size] = flat
                self._remember(slot, entries)
            slot.dev.copy_(slot.host, non_blocking=True)
        slot.copied.record()
        self.last_h2d_bytes = slot.host.numel() * 4
        self._device_tokens(slot.ctx.token_ids, entries, range(len(entries)))
        if slot.pieces is None:
            slot.graph.replay()
        else:
            self._replay_pieces(slot)
        kernels.launch_count += slot.launches    # every replay launches the captured kernels again
        self.graph_replays += 1
        return self._finish(slot.ctx, entries, slot.logits)

    def _capture_pieces(self, slot: _DecodeGraph) -> None:
        """A graph for every capturable run of layers of the model, all from one memory pool. What crosses from one
        piece to the next is the residual stream settled into one float32 tensor: a graph leaves it where the eager
        layers after it read it; eager layers' result is copied to where the graph after them expects it. What comes
        before the first layer (position tables, embedding) and after the last (final norm, head) is always captured:
        as part of the first and last run of layers if those are capturable, else as pieces of their own."""
        ctx, model = slot.ctx, self.model
        layers = len(model.schedule)
        runs = list(self._pieces)
        if not runs[0][2]:
            runs.insert(0, (0, 0, True))
        if not runs[-1][2]:
            runs.append((layers, layers, True))
        pool = torch.cuda.graph_pool_handle()
        slot.pieces = []
        for k, (first, end, capturable) in enumerate(runs):
            piece = _Piece(first, end)
            slot.pieces.append(piece)
            if not capturable:
                continue
            if k > 0:
                piece.inlet = torch.empty((ctx.num_tokens, model.spec.hidden_size), dtype=torch.float32, device=self.device)
            torch.cuda.synchronize(self.device)
            piece.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(piece.graph, pool=pool):
                stream = model.begin(ctx) if k == 0 else ResidualStream(piece.inlet)
                model.run_layers(ctx, self._views, stream, first, end)
                if k + 1 < len(runs):
                    piece.outlet = stream.settle()
                elif ctx.logit_rows is not None:
                    piece.outlet = model.logits(ctx, stream, ctx.logit_rows)
        slot.graph = slot.pieces[0].graph

    def _replay_pieces(self, slot: _DecodeGraph) -> None:
        ctx, model = slot.ctx, self.model
        residual = None
        for piece in slot.pieces:
            if piece.graph is not None:
                if piece.inlet is not None:
                    piece.inlet.copy_(residual)
                piece.graph.replay()
                residual = piece.outlet
                continue
            # eager layers: the step's arrays are the captured step's; what the layers note for themselves is not kept
            eager = copy.copy(ctx)
            eager.memo = {}
            stream = ResidualStream(residual)
            model.run_layers(eager, self._views, stream, piece.first, piece.end)
            residual = stream.settle()
        slot.logits = slot.pieces[-1].outlet

    def _remember(self, slot: _DecodeGraph, entries: Sequence[StepEntry]) -> None:
        slot.req_ids = [(e.req_id, self.cache.admission(e.req_id)) for e in entries]
        slot.table_lens = [[len(self.cache.block_table(e.req_id, g)) for e in entries] for g in range(len(self.cache.groups))]

    def _refill(self, slot: _DecodeGraph, entries: Sequence[StepEntry], width: int) -> None:
        """The same requests as in the slot's last step, one token further: only what moves is written into the
        pinned buffer (token ids, positions, context lengths, the new token's slot, block-table rows that grew or
        belong to a windowed group, whose entries can change in place)."""
        cache, ctx, buf = self.cache, slot.ctx, slot.host_np
        ps = cache.page_size
        R = len(entries)
        starts = [cache.length(e.req_id) for e in entries]
        ctx.starts = starts
        ctx.max_ctx_len = max(starts) + 1
        buf[0:R] = [int(e.tokens[0]) for e in entries]
        buf[R:2 * R] = starts
        at = 3 * R + R + 1                                   # token ids, positions, request of each token, q_start
        buf[at:at + R] = [s + 1 for s in starts]             # ctx_len
        at += 2 * R + ctx.num_logit_rows                     # ctx_len, slots, logit rows
        for g, group in enumerate(cache.groups):
            tables = [cache.block_table(e.req_id, g) for e in entries]
            mapping = []
            for table, start in zip(tables, starts):
                page = table[start // ps]
                mapping.append(-1 if page < 0 else page * ps + start % ps)
            buf[at:at + R] = mapping
            at += R
            lens = slot.table_lens[g]
            windowed = group.spec.window is not None
            for r, table in enumerate(tables):
                if windowed or len(table) != lens[r]:
                    n = min(width, len(table))
                    buf[at + r * width:at + r * width + n] = table[:n]
                    lens[r] = len(table)
            at += R * width
        if self.position_streams > 1:
            for s in range(self.position_streams):
                buf[at:at + R] = [start if e.positions is None else int(e.positions[s][0]) for e, start in zip(entries, starts)]
                at += R

    def _finish(self, ctx: StepContext, entries: Sequence[StepEntry], logits):
        for r, e in enumerate(entries):
            self.cache.commit(e.req_id, ctx.starts[r] + ctx.q_lens[r])
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        return logits

    # -- the step ----------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries as one batch. Returns float32 logits ``[wanted, vocab]`` in the order of
        the entries and of their ``want`` lists, or None when nothing is wanted."""
        entries = list(entries)
        if not entries:
            return None
        with torch.cuda.device(self.device), timing.nvtx_range(f"step of {sum(len(e.tokens) for e in entries)} tokens"):
            if self.use_graphs and all(len(e.tokens) == 1 for e in entries):
                return self._decode_graph_step(entries)
            ctx = self._prepare(entries)
            if self.kernel_times is not None:
                with self.kernel_times:
                    logits = self._run(ctx)
                if len(self.kernel_times.items) > 50000:
                    self.kernel_times.fold()
                return self._finish(ctx, entries, logits)
            return self._finish(ctx, entries, self._run(ctx))

    def release(self, req_id: Hashable) -> None:
        """The request is finished: its pages and slot go back to the pool."""
        if req_id in self.cache:
            self.cache.free(req_id)
