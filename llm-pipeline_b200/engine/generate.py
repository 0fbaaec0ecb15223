"""Generation: requests in, token ids out, through the scheduler, the step function and the sampler.

``GenerationEngine`` is the architecture-neutral engine; ``llm_pipeline_b200.inference`` wraps it
under the reference's names (``Qwen3InferenceEngine``, ``Qwen3InferenceConfig``). One ``step()``
plans a batch (``Scheduler.schedule``), runs it (``ModelRunner.step``) asking for logits only at
the last token of the requests that are due a new token, samples, and records the result. The
reference's loop for one prompt is src/llm_pipeline/inference/qwen3_engine.py:472-550: prefill,
then one token per model call, stopping at EOS or ``max_tokens``.
"""

from __future__ import annotations

import itertools
import os
import time
from dataclasses import dataclass, field, replace
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..cache import CacheManager
from ..config import ModelConfig, load_config
from ..models import Model, build_model, load_model
from ..ops import kernels
from ..sampling import Sampler, SamplingConfig
from .runner import ModelRunner, StepEntry
from .scheduler import PENDING, Request, Scheduler, StepPlan


@dataclass
class GenerationResult:
    req_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: Optional[str]
    preemptions: int = 0
    text: Optional[str] = None


class GenerationEngine:
    def __init__(self, model: Model, config: Optional[ModelConfig] = None, *, page_size: int = 16,
                 num_pages: Optional[int] = None, memory_fraction: float = 0.8, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 2048, max_model_len: Optional[int] = None,
                 max_prefill_chunk: Optional[int] = None, sampling: Optional[SamplingConfig] = None,
                 lookahead: Optional[bool] = None):
        self.model, self.config = model, config
        self.device, self.dtype = model.device, model.dtype
        max_model_len = int(max_model_len or model.spec.max_position)
        specs = model.cache_specs()
        if num_pages is None:
            num_pages = self._pages_that_fit(specs, page_size, memory_fraction, max_num_seqs, max_model_len)
        self.cache = CacheManager(specs, page_size=page_size, num_pages=num_pages, max_requests=max_num_seqs,
                                  max_request_tokens=max_model_len, device=self.device, dtype=self.dtype)
        self.runner = ModelRunner(model, self.cache)
        self.scheduler = Scheduler(self.cache, max_num_seqs, max_num_batched_tokens, max_model_len, max_prefill_chunk)
        self.sampler = Sampler(sampling)
        self._ids = itertools.count()
        self._requests: Dict[Hashable, Request] = {}
        self.lookahead = os.environ.get("LLMP_B200_LOOKAHEAD", "1") != "0" if lookahead is None else bool(lookahead)
        self._in_flight = None                   # (sampled ids on the device, their requests, their landing place) of the step not read back yet
        self._landing: list = []                 # pinned host buffers with an event each, for the sampled ids' way to the host
        self.steps = 0
        self.tokens_prefilled = 0
        self.tokens_decoded = 0

    @classmethod
    def from_folder(cls, model_dir: str, device: str = "cuda:0", dtype: torch.dtype = torch.bfloat16, **kwargs):
        config, model = load_model(model_dir, device, dtype)
        return cls(model, config, **kwargs)

    def _pages_that_fit(self, specs, page_size: int, fraction: float, max_num_seqs: int, max_model_len: int) -> int:
        """Pages per group from the device memory that is free after the weights: ``fraction`` of it,
        capped at what ``max_num_seqs`` requests of ``max_model_len`` tokens can use."""
        per_page = sum(CacheManager.bytes_per_page(specs, page_size, self.dtype))      # one page id in every group
        if per_page == 0:
            return 1
        free, _total = torch.cuda.mem_get_info(self.device)
        cap = max_num_seqs * -(-max_model_len // page_size)
        return max(1, min(cap, int(free * fraction) // per_page))

    # -- requests --------------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], max_tokens: int = 16,
                    sampling: Optional[SamplingConfig] = None, eos_token_ids: Optional[Sequence[int]] = None,
                    ignore_eos: bool = False, req_id: Optional[Hashable] = None,
                    position_ids: Optional[Sequence[Sequence[int]]] = None) -> Hashable:
        """``position_ids``: for a model whose position encoding reads several streams of positions, the prompt's
        position ids, one sequence per stream (see ``Request.position_ids``)."""
        req_id = next(self._ids) if req_id is None else req_id
        if req_id in self._requests and self._requests[req_id].status != "finished":
            raise ValueError(f"request id {req_id!r} is in use")
        for t in prompt_token_ids:
            if not 0 <= int(t) < self.model.spec.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary of {self.model.spec.vocab_size}")
        if eos_token_ids is None:
            eos_token_ids = self.config.eos_token_ids() if self.config is not None else []
        streams = self.runner.position_streams
        if position_ids is not None and (len(position_ids) != streams or any(len(row) != len(prompt_token_ids) for row in position_ids)):
            raise ValueError(f"position ids must be [{streams}][{len(prompt_token_ids)}]: one row for each stream of the "
                             "model's position encoding, one id for each prompt token")
        request = Request(req_id, [int(t) for t in prompt_token_ids], sampling or self.sampler.config,
                          int(max_tokens), set(int(t) for t in eos_token_ids), ignore_eos,
                          position_ids=None if position_ids is None else [[int(x) for x in row] for row in position_ids])
        self.scheduler.add(request)
        self._requests[req_id] = request
        return req_id

    def has_unfinished(self) -> bool:
        # (ids still in flight for requests that are all finished, stopped or aborted meanwhile, are nobody's business)
        return self.scheduler.has_unfinished() or (self._in_flight is not None and
                                                   any(r.status != "finished" for r in self._in_flight[1]))

    # -- one step --------------------------------------------------------------------------
    def step(self) -> List[Request]:
        """Plan and launch one batch, then read back what the batch before it sampled; returns the requests that are
        finished with all their tokens known.

        The engine runs one step ahead of what it has read (``lookahead``): a step's sampled ids stay on the device,
        the next step takes them from there (``StepEntry.device_token``) and is planned and queued while the device
        still works on this one; only then does the host wait for this step's ids. So the device never waits for the
        host between steps. What the plan of the next step needs of a token it cannot see is only that it exists
        (``Request.in_flight``); a request that an end-of-sequence token ends was then planned one step too far, and
        what that step sampled for it is dropped. A request with a repetition penalty needs its tokens on the host
        before the next is sampled: while one is running or waiting, every step is read back before the next is planned."""
        finished: List[Request] = []
        ahead = self.lookahead and not any(r.sampling.repetition_penalty != 1.0
                                           for r in list(self.scheduler.running) + list(self.scheduler.waiting))
        if not ahead:
            finished += self._read_back()
        plan: StepPlan = self.scheduler.schedule()
        finished += plan.aborted
        if not plan.entries:
            if self._in_flight is not None:
                return finished + self._read_back()
            if not finished and self.scheduler.has_unfinished():
                raise RuntimeError("the scheduler could not plan a step although requests are unfinished")
            return finished
        entries = []
        source, where = None, {}
        if self._in_flight is not None:
            source = self._in_flight[0]
            where = {id(request): row for row, request in enumerate(self._in_flight[1])}
        for e in plan.entries:
            tokens, on_device = e.token_ids, None
            if tokens[-1] == PENDING:
                # the id is among those the step before sampled
                on_device = (source, where[id(e.request)])
                tokens = [0]
                if e.count != 1:
                    raise RuntimeError("a token that is still on the device can only be a step's single token")
            entries.append(StepEntry(e.request.req_id, tokens, [e.count - 1] if e.samples else [], e.positions, on_device))
        logits = self.runner.step(entries)
        due = [e for e in plan.entries if e.samples]
        launched = None
        if due:
            tokens = self.sampler.sample_rows(
                logits, [e.request.sampling for e in due], [len(e.request.output) + e.request.in_flight for e in due],
                [e.request.output if e.request.sampling.repetition_penalty != 1.0 else None for e in due])
            # to the host at once, behind this step and before the next is queued: reading it back later then waits
            # for this step only (a copy asked for later would queue behind the step after it)
            landing = self._landing.pop() if self._landing else (torch.empty(self.scheduler.max_num_seqs, dtype=torch.int32).pin_memory(),
                                                                 torch.cuda.Event())
            landing[0][:tokens.numel()].copy_(tokens, non_blocking=True)
            landing[1].record()
            launched = (tokens, [e.request for e in due], landing)
        self.steps += 1
        for e in plan.entries:
            if e.count == 1 and (e.request.output or e.request.in_flight):
                self.tokens_decoded += 1
            else:
                self.tokens_prefilled += e.count
        finished += self.scheduler.finish_step(plan, {e.request.req_id: None for e in due})
        # the step before: its ids are on their way or there; this step is queued behind it
        finished += self._read_back()
        self._in_flight = launched
        if not ahead:
            finished += self._read_back()
        return finished

    def abort(self, req_id: Hashable) -> Optional[Request]:
        """Take the request out wherever it is; its pages go back. What is still in flight for it is dropped."""
        request = self.scheduler.abort(req_id)
        if request is None:
            request = self._requests.get(req_id)
            if request is None or request.status != "draining":
                return None
            request.status, request.finish_reason = "finished", "abort"     # its last token was on its way
        return request

    def drain(self) -> List[Request]:
        """Read back what is in flight without launching anything; returns the requests this finishes."""
        return self._read_back()

    def _read_back(self) -> List[Request]:
        """The sampled ids of the step in flight, to the host and into their requests."""
        if self._in_flight is None:
            return []
        tokens, requests, landing = self._in_flight
        self._in_flight = None
        finished = []
        landing[1].synchronize()
        values = landing[0][:len(requests)].tolist()
        self._landing.append(landing)
        for request, token in zip(requests, values):
            if self.scheduler.late_token(request, token):
                finished.append(request)
        kernels.check_error_flag()                      # after the copy above: the step's kernels have run
        return finished

    # -- whole generations -------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 16, temperature: Optional[float] = None,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, seed: Optional[int] = None,
                 ignore_eos: bool = False, **sampling_overrides) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids); results in the order of the prompts.
        Prompt i samples with seed ``seed + i``."""
        base = self.sampler.config.merged({"temperature": temperature, "top_k": top_k, "top_p": top_p,
                                           **sampling_overrides})
        first_seed = base.seed if seed is None else int(seed)
        ids = [self.add_request(p, max_tokens, replace(base, seed=first_seed + i), ignore_eos=ignore_eos)
               for i, p in enumerate(prompts)]
        while any(self._requests[i].status != "finished" for i in ids):
            self.step()
        results = []
        for i in ids:
            r = self._requests.pop(i)
            results.append(GenerationResult(i, r.prompt, r.output, r.finish_reason, r.preemptions))
        return results

    def stats(self) -> Dict[str, object]:
        out = {"steps": self.steps, "tokens_prefilled": self.tokens_prefilled, "tokens_decoded": self.tokens_decoded}
        out.update(self.scheduler.stats())
        out.update(self.cache.stats())
        if self.runner.kernel_times is not None:             # LLMP_B200_KERNEL_TIMES=1
            out["kernel_times"] = self.runner.kernel_times.table()
        return out
