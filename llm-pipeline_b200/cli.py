"""Command line in the manner of the reference's ``llm-pipeline infer``
(src/llm_pipeline/cli.py:97-133): ``python -m llm_pipeline_b200.cli infer --model DIR --prompt TEXT
[--device cuda:0] [--dtype bf16|fp32] [--max-new-tokens 256] [--temperature 0.7] [--chat]``.
``--prompt-ids`` takes token ids instead of text (for model folders without a tokenizer); ``fp16``
is accepted as a choice, as there, but refused with a message: this engine computes in bf16 or
fp32. ``random-model`` writes a model folder with seeded random weights; ``replay`` is the trace
replay of ``bin/trace_run``. The reference's ``serve``, ``train`` and ``merge`` are not part of
this engine."""

from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def _cmd_infer(args: argparse.Namespace) -> int:
    from .inference import Qwen3InferenceConfig, Qwen3InferenceEngine

    if args.dtype == "fp16":
        print("fp16 is not built into this engine; use --dtype bf16 or fp32", file=sys.stderr)
        return 2
    if (args.prompt is None) == (args.prompt_ids is None):
        print("give exactly one of --prompt and --prompt-ids", file=sys.stderr)
        return 2
    engine = Qwen3InferenceEngine(Qwen3InferenceConfig(
        model_path=args.model, device=args.device, dtype=args.dtype, max_new_tokens=args.max_new_tokens,
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed,
        block_size=args.block_size, num_blocks=args.num_blocks, max_sequence_length=args.max_sequence_length,
        max_num_batched_tokens=args.max_num_batched_tokens))
    if args.prompt_ids is not None:
        prompt = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
        out = engine.generate(prompt, max_tokens=args.max_new_tokens, temperature=args.temperature)
        print(" ".join(str(t) for t in out))
        return 0
    text = args.prompt
    if args.chat:
        if engine.tokenizer is None:
            print("--chat needs a tokenizer in the model folder", file=sys.stderr)
            return 2
        text = engine.tokenizer.apply_chat_template([{"role": "user", "content": args.prompt}], tokenize=False,
                                                    add_generation_prompt=True)
    out = engine.generate(text, max_tokens=args.max_new_tokens, temperature=args.temperature)
    print(out if isinstance(out, str) else "\n---\n".join(out))
    return 0


def _cmd_random_model(args: argparse.Namespace) -> int:
    import torch

    from .weights import write_random_model

    with open(args.config) as f:
        config = json.load(f)
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32}[args.dtype]
    print(write_random_model(config, args.seed, args.out, dtype=dtype, std=args.std))
    return 0


def _cmd_replay(args: argparse.Namespace) -> int:
    from .replay import main as replay_main

    return replay_main(["--model", args.model, "--dtype", args.dtype, "--out", args.out, "--max-tokens",
                        str(args.max_tokens), "--device", args.device])


def main(argv: Optional[List[str]] = None) -> int:
    parser = argparse.ArgumentParser(prog="llm-pipeline-b200")
    sub = parser.add_subparsers(dest="cmd", required=True)

    p = sub.add_parser("infer", help="One-off generation")
    p.add_argument("--model", required=True)
    p.add_argument("--prompt")
    p.add_argument("--prompt-ids", help="token ids separated by spaces or commas, instead of --prompt")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="bf16", choices=("fp16", "bf16", "fp32"))
    p.add_argument("--max-new-tokens", type=int, default=256)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--chat", action="store_true", help="Wrap prompt in chat template")
    p.add_argument("--top-k", type=int, default=50)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--num-blocks", type=int, default=None)
    p.add_argument("--max-sequence-length", type=int, default=2048)
    p.add_argument("--max-num-batched-tokens", type=int, default=2048)
    p.set_defaults(fn=_cmd_infer)

    p = sub.add_parser("random-model", help="Write a model folder with seeded random weights")
    p.add_argument("--config", required=True, help="a config.json of the architecture")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--out", required=True)
    p.add_argument("--dtype", default="bf16", choices=("bf16", "fp32"))
    p.add_argument("--std", type=float, default=0.02)
    p.set_defaults(fn=_cmd_random_model)

    p = sub.add_parser("replay", help="Feed token ids step by step (JSON lines on stdin) and write logits")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True)
    p.add_argument("--device", default="cuda:0")
    p.set_defaults(fn=_cmd_replay)

    args = parser.parse_args(argv)
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    raise SystemExit(main())
