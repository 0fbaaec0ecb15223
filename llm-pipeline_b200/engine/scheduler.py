"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

The reference's ``ContinuousBatcher`` admits from a FIFO queue while fewer than ``max_batch_size``
requests are active (src/llm_pipeline/inference/continuous_batching.py:346-360), right-pads all
active requests into one rectangle and re-runs every prompt from scratch whenever a request joins
or leaves (:104,115,372-378); a request is finished by its EOS token or by ``max_tokens`` (:68-81)
and its pages are freed on completion (:417-446). There is no token budget and no partial prompt.
Here every step is planned under ``max_num_batched_tokens``: first one token for each request that
is decoding, then portions of prompts (requests that are part-way through theirs first, then new
admissions in arrival order), each portion at most ``max_prefill_chunk`` tokens.

When pages run out (decided here, because the cache manager never evicts):
* a waiting request is simply not admitted yet, and no request behind it overtakes it;
* if a running request cannot get the page its next tokens need, the request admitted last is
  preempted: its pages and slot are freed and it returns to the front of the waiting queue to be
  recomputed from its prompt plus what it has generated; nothing is admitted in that step;
* if the only running request cannot get a page, it is finished with reason ``"out_of_pages"``.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Set

from ..cache import CacheManager
from ..sampling import SamplingConfig


PENDING = -1                  # stands for a sampled token that is still on the device (``Request.in_flight``)


@dataclass(eq=False)          # a request is itself: lists of requests are searched by identity, not by comparing fields
class Request:
    req_id: Hashable
    prompt: List[int]
    sampling: SamplingConfig
    max_tokens: int
    eos_token_ids: Set[int] = field(default_factory=set)
    ignore_eos: bool = False
    output: List[int] = field(default_factory=list)
    computed: int = 0                  # tokens whose keys/values are in the cache
    status: str = "waiting"            # waiting | running | draining | finished
    # Tokens that were sampled for this request in steps whose result has not reached the host yet (the engine runs
    # one step ahead of what it has read back). They count as tokens of the request everywhere, but ``output`` holds
    # only tokens the host knows. "draining": the request has left the scheduler (its last token is among these).
    in_flight: int = 0
    finish_reason: Optional[str] = None
    preemptions: int = 0
    # For a model whose position encoding reads several streams of positions: the prompt's position ids, one list per
    # stream. Generated tokens go on from the largest position id of the prompt, by one per token, in every stream.
    position_ids: Optional[List[List[int]]] = None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output + [PENDING] * self.in_flight

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output) + self.in_flight

    def token_slice(self, start: int, count: int) -> List[int]:
        """``tokens[start:start + count]`` without putting the whole list together (a decode step asks for one token
        of every request, step after step)."""
        n, end = len(self.prompt), start + count
        if end <= n:
            return self.prompt[start:end]
        known = n + len(self.output)
        out = self.prompt[start:] if start < n else []
        if start < known:
            out = out + self.output[max(start - n, 0):min(end, known) - n]
        if end > known:
            out = out + [PENDING] * (min(end, known + self.in_flight) - max(start, known))
        return out

    def positions_of(self, start: int, count: int) -> Optional[List[List[int]]]:
        """Position ids of the tokens start .. start + count - 1, stream by stream; None without ``position_ids``."""
        if self.position_ids is None:
            return None
        n = len(self.prompt)
        after = 1 + max(max(row) for row in self.position_ids) if n else 0
        tail = [after + i - n for i in range(max(start, n), start + count)]
        return [list(row[start:min(start + count, n)]) + tail for row in self.position_ids]

    @property
    def num_pending(self) -> int:
        return len(self.prompt) + len(self.output) + self.in_flight - self.computed


@dataclass
class PlannedEntry:
    request: Request
    start: int          # first token of the portion (= request.computed)
    count: int          # tokens in the portion
    samples: bool       # the portion reaches the request's last token, so a token is sampled

    @property
    def token_ids(self) -> List[int]:
        return self.request.token_slice(self.start, self.count)

    @property
    def positions(self) -> Optional[List[List[int]]]:
        return self.request.positions_of(self.start, self.count)


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    aborted: List[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int, max_prefill_chunk: Optional[int] = None):
        if max_num_batched_tokens < 1 or max_num_seqs < 1:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be at least 1")
        self.cache = cache
        self.max_num_seqs = min(int(max_num_seqs), cache.max_requests)
        self.max_num_batched_tokens = int(max_num_batched_tokens)
        self.max_model_len = min(int(max_model_len), cache.max_request_tokens)
        self.max_prefill_chunk = int(max_prefill_chunk or max_num_batched_tokens)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []       # in order of admission
        self.num_preemptions = 0
        self.num_finished = 0

    # -- requests --------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.req_id!r} has an empty prompt")
        if len(request.prompt) >= self.max_model_len:
            raise ValueError(f"request {request.req_id!r}: a prompt of {len(request.prompt)} tokens leaves no room "
                             f"to generate within {self.max_model_len} tokens")
        if request.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        request.status = "waiting"
        self.waiting.append(request)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # -- planning one step -------------------------------------------------------------------
    def _release(self, request: Request) -> None:
        if request.req_id in self.cache:
            self.cache.free(request.req_id)

    def _preempt_last(self, plan: StepPlan) -> Request:
        victim = self.running.pop()
        self._release(victim)
        victim.computed = 0
        victim.status = "waiting"
        victim.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)
        plan.entries = [e for e in plan.entries if e.request is not victim]
        return victim

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_num_batched_tokens
        spare = [0] * len(self.cache.groups)

        def try_plan(request: Request, limit: int) -> bool:
            nonlocal budget, spare
            count = min(request.num_pending, budget, limit)
            if count <= 0:
                return False
            new_length = request.computed + count
            short = self.cache.pages_short(request.req_id, new_length)
            if not self.cache.can_reserve(request.req_id, new_length, spare, short):
                return False
            if any(short):
                spare = [a + b for a, b in zip(spare, short)]
            budget -= count
            plan.entries.append(PlannedEntry(request, request.computed, count, request.computed + count == request.num_tokens))
            return True

        # 1. running requests: those that decode first, then those still in their prompt
        order = [r for r in self.running if r.num_pending == 1] + [r for r in self.running if r.num_pending > 1]
        for request in order:
            if request.status != "running":      # preempted while planning an earlier one
                continue
            while budget > 0:
                limit = 1 if request.num_pending == 1 else self.max_prefill_chunk
                if try_plan(request, limit):
                    break
                # no pages: make room by preempting the request admitted last
                if len(self.running) == 1:
                    self.running.remove(request)
                    self._release(request)
                    request.status, request.finish_reason = "finished", "out_of_pages"
                    self.num_finished += 1
                    plan.aborted.append(request)
                    break
                victim = self._preempt_last(plan)
                # pages planned for the victim in this step are free again
                budget = self.max_num_batched_tokens - plan.num_tokens
                spare = [0] * len(self.cache.groups)
                for e in plan.entries:
                    short = self.cache.pages_short(e.request.req_id, e.start + e.count)
                    spare = [a + b for a, b in zip(spare, short)]
                if victim is request:
                    break
        # 2. admissions, in arrival order, only when nothing was preempted in this step
        if not plan.preempted:
            admitted = 0
            while (self.waiting and budget > 0 and len(self.running) < self.max_num_seqs
                   and self.cache.free_slots - admitted > 0):
                request = self.waiting[0]
                if not try_plan(request, self.max_prefill_chunk):
                    if not self.running and not plan.entries:
                        # nothing runs and the head of the queue still cannot start: it never will
                        self.waiting.popleft()
                        request.status, request.finish_reason = "finished", "out_of_pages"
                        self.num_finished += 1
                        plan.aborted.append(request)
                        continue
                    break
                self.waiting.popleft()
                request.status = "running"
                self.running.append(request)
                admitted += 1
        return plan

    # -- after the step ran ------------------------------------------------------------------
    def finish_step(self, plan: StepPlan, sampled: Dict[Hashable, Optional[int]]) -> List[Request]:
        """Record the step: portions are now cached, sampled tokens are appended, finished requests
        leave and give their pages back. Returns the requests that finished. A token given as None was
        sampled but has not reached the host (``late_token`` brings it): it counts towards the lengths,
        and a request whose last token it is leaves the scheduler as "draining"."""
        finished: List[Request] = []
        for entry in plan.entries:
            request = entry.request
            request.computed = entry.start + entry.count
            if not entry.samples:
                continue
            token = sampled[request.req_id]
            reason = None
            if token is None:
                request.in_flight += 1
            else:
                request.output.append(int(token))
                if not request.ignore_eos and int(token) in request.eos_token_ids:
                    reason = "stop"
            generated = len(request.output) + request.in_flight
            if reason is None and (generated >= request.max_tokens or len(request.prompt) + generated >= self.max_model_len):
                reason = "length"
            if reason:
                request.finish_reason = reason
                self.running.remove(request)
                self._release(request)
                self.num_finished += 1
                if request.in_flight:
                    request.status = "draining"
                else:
                    request.status = "finished"
                    finished.append(request)
        return finished

    def late_token(self, request: Request, token: int) -> bool:
        """The oldest of the request's tokens in flight has reached the host. True when the request is finished by it:
        it was the last one of a draining request, or it ends the request (an end-of-sequence token; what was computed
        for the request after it was computed in vain and is dropped when it arrives)."""
        request.in_flight -= 1
        if request.status == "finished":
            return False                           # stopped or aborted before this token: dropped
        token = int(token)
        request.output.append(token)
        if not request.ignore_eos and token in request.eos_token_ids:
            if request.status == "running":
                self.running.remove(request)
                self._release(request)
                self.num_finished += 1
            elif request.status == "waiting":      # preempted with the token in flight
                self.waiting.remove(request)
                self.num_finished += 1
            request.status, request.finish_reason = "finished", "stop"
            return True
        if request.status == "draining" and request.in_flight == 0:
            request.status = "finished"
            return True
        return False

    def abort(self, req_id: Hashable) -> Optional[Request]:
        for request in list(self.running):
            if request.req_id == req_id:
                self.running.remove(request)
                self._release(request)
                request.status, request.finish_reason = "finished", "abort"
                return request
        for request in list(self.waiting):
            if request.req_id == req_id:
                self.waiting.remove(request)
                request.status, request.finish_reason = "finished", "abort"
                return request
        return None

    def stats(self) -> Dict[str, int]:
        return {"waiting": len(self.waiting), "running": len(self.running),
                "preemptions": self.num_preemptions, "finished": self.num_finished}
