"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and owns no model code: it loads the model the way generation does, makes a
cache pool for ``--max-tokens`` tokens and calls the engine's step function once per input line.

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits are wanted;
all entries of a step run as one batch. ``end``: requests that are finished after this step; their
pages and slot are given back. For a step in which something is wanted, ``<out>/<step>.f32``
receives the logits ``[wanted, vocab]`` as little-endian float32 in the order of the entries and
of ``want``. Every step that brings entries also writes ``<out>/<step>.pages.json``: for each of its requests the
page ids of its block table in every cache group after the step (-1: a page a window has passed), so that a reader
can see from the files alone that a page went from a finished request to a later one. After every step the line
``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional, Sequence

PAGE_SIZE = 16          # tokens per page; divides the 64-token rounding of --max-tokens
MAX_LIVE_REQUESTS = 64  # state slots (a trace keeps at most a handful of requests live)


def main(argv: Optional[Sequence[str]] = None, stdin=None, stdout=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout

    import torch

    from .cache import CacheManager
    from .engine import ModelRunner, StepEntry
    from .models import load_model
    from .ops import build_library, kernels

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine has no CPU path", file=sys.stderr)
        return 3
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    build_library()
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    _config, model = load_model(args.model, args.device, dtype)
    max_tokens = max(64, -(-args.max_tokens // 64) * 64)
    cache = CacheManager(model.cache_specs(), page_size=PAGE_SIZE, num_pages=max_tokens // PAGE_SIZE,
                         max_requests=MAX_LIVE_REQUESTS, max_request_tokens=max_tokens,
                         device=model.device, dtype=dtype)
    runner = ModelRunner(model, cache)
    os.makedirs(args.out, exist_ok=True)

    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in record.get("entries", [])]
        logits = runner.step(entries) if entries else None
        if logits is not None:
            logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4").tofile(
                os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize(model.device)
        if entries:
            tables = {str(e.req_id): [list(cache.block_table(e.req_id, g)) for g in range(len(cache.groups))] for e in entries}
            with open(os.path.join(args.out, f"{step}.pages.json"), "w") as f:
                json.dump({"step": step, "page_size": PAGE_SIZE, "pages": tables}, f)
        kernels.check_error_flag()                      # a kernel whose bounded wait ran out leaves no valid logits
        for req_id in record.get("end", []):
            runner.release(req_id)
        print(f"done {step}", file=stdout, flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
