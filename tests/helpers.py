"""Helpers shared by the GPU tests: model folders from the plain implementation's random weights,
engines over them, and the ways of cutting a set of requests into steps."""

from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence, Tuple

import torch

import plain_qwen3 as plain

# absolute, on logits of the tiny models (largest about 1); the engine in bfloat16 is about 5e-3 from the oracle there
TOL = {torch.float32: 1e-4, torch.bfloat16: 1.5e-2}


def write_model_dir(path: str, config: dict, weights: Dict[str, torch.Tensor], dtype: torch.dtype) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f)
    return path


def make_case(tmp_path, config: dict, seed: int, dtype: torch.dtype, std: float = 0.02):
    """(model folder, weights as the engine sees them in float32)."""
    weights = plain.random_weights(config, seed, std=std)
    if dtype == torch.bfloat16:
        weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    folder = write_model_dir(str(tmp_path), config, weights, dtype)
    return folder, weights


def make_runner(folder: str, dtype: torch.dtype, page_size: int, num_pages: int, max_request_tokens: int = 4096,
                max_requests: int = 8):
    from llm_pipeline_b200.cache import CacheManager
    from llm_pipeline_b200.engine import ModelRunner
    from llm_pipeline_b200.models import load_model

    _config, model = load_model(folder, "cuda:0", dtype)
    cache = CacheManager(model.cache_specs(), page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                         max_request_tokens=max_request_tokens, device=model.device, dtype=dtype)
    return ModelRunner(model, cache)


def random_tokens(vocab: int, length: int, seed: int) -> List[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()


# A trace is a list of steps; a step is (entries, end) with entries = [(req_id, tokens, want)].
Step = Tuple[List[Tuple[str, List[int], List[int]]], List[str]]


def cut_whole(requests: Dict[str, List[int]]) -> List[Step]:
    return [([(rid, toks, list(range(len(toks))))], [rid]) for rid, toks in requests.items()]


def cut_tail_one_by_one(requests: Dict[str, List[int]], tail: int = 32) -> List[Step]:
    steps: List[Step] = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append(([(rid, toks[:head], list(range(head)))], []))
        for i in range(head, len(toks)):
            steps.append(([(rid, [toks[i]], [0])], []))
        steps[-1] = (steps[-1][0], [rid])
    return steps


def cut_portions(requests: Dict[str, List[int]], sizes: Sequence[int]) -> List[Step]:
    steps: List[Step] = []
    k = 0
    for rid, toks in requests.items():
        done = 0
        while done < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - done)
            k += 1
            steps.append(([(rid, toks[done:done + n], list(range(n)))], []))
            done += n
        steps[-1] = (steps[-1][0], [rid])
    return steps


def cut_mixed(requests: Dict[str, List[int]], sizes: Sequence[int], max_live: int = 4, decode_tail: int = 6) -> List[Step]:
    """Up to ``max_live`` requests at a time: each advances by a portion of changing size while it is
    in its prompt part and by single tokens over its last ``decode_tail`` tokens; a finished request
    ends and the next one starts, so its pages are handed to a later request."""
    waiting = list(requests.items())
    live: List[Tuple[str, List[int], int]] = []
    steps: List[Step] = []
    k = 0
    tick = 0
    while waiting or live:
        tick += 1
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append((rid, toks, 0))
        entries, end, nxt = [], [], []
        for i, (rid, toks, done) in enumerate(live):
            if (tick + i) % 5 == 4 and done > 0:      # now and then a request sits a step out
                nxt.append((rid, toks, done))
                continue
            remaining = len(toks) - done
            if remaining <= decode_tail:
                n = 1
            else:
                n = min(sizes[k % len(sizes)], remaining - decode_tail)
                k += 1
            entries.append((rid, toks[done:done + n], list(range(n))))
            done += n
            if done == len(toks):
                end.append(rid)
            else:
                nxt.append((rid, toks, done))
        live = nxt
        if entries:
            steps.append((entries, end))
    return steps


def replay(runner, steps: List[Step]) -> Dict[str, torch.Tensor]:
    """Run the steps through the engine's step function; logits per request in token order."""
    from llm_pipeline_b200.engine import StepEntry

    rows: Dict[str, List[torch.Tensor]] = {}
    for entries, end in steps:
        logits = runner.step([StepEntry(rid, toks, want) for rid, toks, want in entries])
        cursor = 0
        for rid, _toks, want in entries:
            rows.setdefault(rid, []).append(logits[cursor:cursor + len(want)].float().cpu())
            cursor += len(want)
        for rid in end:
            runner.release(rid)
        runner.cache.check()
    return {rid: torch.cat(parts) for rid, parts in rows.items()}


def expected_logits(config: dict, weights: Dict[str, torch.Tensor], requests: Dict[str, List[int]]):
    return {rid: plain.forward_logits(config, weights, toks) for rid, toks in requests.items()}


def assert_close(got: Dict[str, torch.Tensor], want: Dict[str, torch.Tensor], tol: float, what: str):
    for rid, ref in want.items():
        assert got[rid].shape == ref.shape, f"{what}: request {rid} has shape {tuple(got[rid].shape)}, expected {tuple(ref.shape)}"
        diff = (got[rid] - ref).abs()
        worst = float(diff.max())
        if not worst <= tol:
            pos = int(diff.max(dim=1).values.argmax())
            raise AssertionError(f"{what}: request {rid}: max |logit difference| {worst:.3e} > {tol:.1e}; "
                                 f"first position above tolerance: {int((diff.max(dim=1).values > tol).nonzero()[0])}, "
                                 f"worst position {pos} of {ref.shape[0]}")
