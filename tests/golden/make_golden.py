"""Compare the plain implementation once with the reference's own model code on the CPU.

Usage:  python tests/golden/make_golden.py /path/to/llm-pipeline

It loads ``src/llm_pipeline/models/qwen3/custom_builder.py`` of DavidAkinpelu/llm-pipeline by
file path (that file imports only torch), builds ``Qwen3ForCausalLM`` for the tiny configurations
of ``tests/plain_qwen3.py``, loads the same seeded random weights by name, and runs in float32:

* one forward over a whole sequence, and
* the reference's own incremental path (a prefix, then single tokens with ``past_key_values``).

It prints the largest differences from ``plain_qwen3.forward_logits`` and writes
``tests/golden/<name>.json``: the token ids and, for a few positions, the reference's logits over
the whole vocabulary, its argmax and the largest absolute logit, so that
``tests/test_plain_reference.py`` can check the plain implementation without the reference. All five
tiny configurations are recorded, head sizes 16, 32, 48, 64 and 128 among them.
"""

from __future__ import annotations

import importlib.util
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_qwen3 as plain  # noqa: E402


def load_reference(root: str):
    path = os.path.join(root, "src", "llm_pipeline", "models", "qwen3", "custom_builder.py")
    spec = importlib.util.spec_from_file_location("reference_custom_builder", path)
    module = importlib.util.module_from_spec(spec)
    sys.dont_write_bytecode = True
    spec.loader.exec_module(module)
    return module


def main() -> int:
    if len(sys.argv) < 2:
        print("usage: make_golden.py <checkout of DavidAkinpelu/llm-pipeline>", file=sys.stderr)
        return 2
    root = sys.argv[1]
    ref = load_reference(root)
    torch.manual_seed(0)
    summary = {}
    for name, config, seed, length in (("tiny_a", plain.TINY_A, 0, 33), ("tiny_b", plain.TINY_B, 1, 40),
                                       ("tiny_c", plain.TINY_C, 2, 29), ("tiny_d", plain.TINY_D, 3, 37),
                                       ("tiny_e", plain.TINY_E, 4, 45)):
        weights = plain.random_weights(config, seed)
        model = ref.Qwen3ForCausalLM(ref.Qwen3Config(**config)).eval()
        state = dict(weights)
        if config["tie_word_embeddings"]:
            state["lm_head.weight"] = weights["model.embed_tokens.weight"]
        missing, unexpected = model.load_state_dict(state, strict=False)
        assert not unexpected, unexpected
        assert all("inv_freq" in m for m in missing), missing
        gen = torch.Generator().manual_seed(100 + seed)
        ids = torch.randint(0, config["vocab_size"], (length,), generator=gen).tolist()
        with torch.no_grad():
            whole = model(input_ids=torch.tensor([ids])).logits[0]
            prefix = length - 8
            out = model(input_ids=torch.tensor([ids[:prefix]]), use_cache=True)
            rows = [out.logits[0]]
            past = out.past_key_values
            for token in ids[prefix:]:
                out = model(input_ids=torch.tensor([[token]]), past_key_values=past, use_cache=True)
                rows.append(out.logits[0])
                past = out.past_key_values
            incremental = torch.cat(rows, dim=0)
        mine = plain.forward_logits(config, weights, ids)
        diff_whole = float((mine - whole).abs().max())
        diff_incremental = float((mine - incremental).abs().max())
        scale = float(whole.abs().max())
        print(f"{name}: max|plain - reference whole| = {diff_whole:.3e}, "
              f"max|plain - reference incremental| = {diff_incremental:.3e}, max|logit| = {scale:.3f}")
        positions = [0, 1, length // 2, length - 1]
        summary = {
            "config": config, "seed": seed, "token_ids": ids, "positions": positions,
            "logits": [[round(float(v), 7) for v in whole[p]] for p in positions],
            "argmax": [int(whole[p].argmax()) for p in positions],
            "max_abs_logit": scale,
            "plain_minus_reference_whole": diff_whole,
            "plain_minus_reference_incremental": diff_incremental,
        }
        with open(os.path.join(HERE, f"{name}.json"), "w") as f:
            f.write("{\n" + ",\n".join(f" {json.dumps(k)}: {json.dumps(v)}" for k, v in summary.items()) + "\n}\n")
        assert diff_whole < 2e-5 and diff_incremental < 5e-5
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
