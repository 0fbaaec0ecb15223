"""Serving benchmark on one B200: decode tokens per second of a Qwen3-8B-shaped model.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

The default run has the layer sizes of the Qwen3-8B configuration (36 layers, hidden 4096, 32 query
and 8 key/value heads of 128, intermediate 12288, vocabulary 151936) with random bfloat16 weights,
a batch of 8 requests and 2,048 tokens of context each. A "step" is one decode step: one new token
for every request of the batch, from the embedding to the sampled token id. It prints one JSON line:
``value`` is decoded tokens per second timed on the device with CUDA events; ``e2e`` is the same
through the Python entry point (``GenerationEngine.step``: host token lists in, host token ids out,
the index arrays copied from pinned memory every step); ``prefill`` is one 2,048-token prompt in one
step; ``roofline`` is the decode step against the bytes it must read; ``points`` are decode at batch
1 and 64, at batch 8 with pages of 32 tokens, and two further sizes at their full depth (the Qwen3-0.6B shape under a
continuous-batching mix of 64 requests, decode at batch 8 at the Qwen3-32B shape). ``breakdown`` gives, for one decode step of the batch
and for the prefill step, the device time of every kernel class (CUDA events around every launch of
an eager step that is queued behind a sleeping kernel, so that launches do not wait for the host) with
the achieved GB/s of the weight-streaming products and the decode attention and the TFLOP/s of the
prefill products and attention, each over the measured peak (burst figure: kernels alone).
``baselines.plain_pytorch`` is this repository's plain PyTorch implementation (``tests/plain_qwen3.py``:
whole sequences, no cache) on the same GPU in bfloat16 at batch 1. ``selfcheck`` compares, outside any
timed region, the greedy tokens of steps of 8 and 64 requests on a two-layer model of the same widths
with the plain implementation. All weights and token ids are synthetic (seeded); the inputs are far
larger than L2, so no flush is needed between iterations.

``--impl reference`` runs DavidAkinpelu/llm-pipeline's own ``Qwen3ForCausalLM`` from
``baseline/_ref`` (installed offline with pip --no-deps --target) with its ``past_key_values``
loop at the same sizes and prints the same line with ``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 4096, "hidden_act": "silu",
}
QWEN3_0_6B = {**QWEN3_8B, "num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16, "num_key_value_heads": 8,
              "intermediate_size": 3072, "tie_word_embeddings": True}
QWEN3_32B = {**QWEN3_8B, "num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "num_key_value_heads": 8,
             "intermediate_size": 25600}
SHAPES = {"8b": ("Qwen3-8B shape", QWEN3_8B), "0.6b": ("Qwen3-0.6B shape", QWEN3_0_6B), "32b": ("Qwen3-32B shape", QWEN3_32B)}
CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE_SIZE = 16           # tokens per page of the key/value cache (--page-size)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            return {"hbm_gbs": float(data["hbm_gbs"]),
                    "bf16_tflops": float(data.get("bf16_tflops_sustained") or data["bf16_tflops"]),
                    "bf16_tflops_burst": float(data["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons, max_clock = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(int(float(parts[0])))
                max_clock = int(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def weight_bytes(cfg, layers, element=2):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d, nq, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I + 2 * H + 2 * d
    return (layers * per_layer + V * H + H) * element          # the layers, the output head and the final norm


def kv_bytes_per_token(engine):
    """Bytes the caches of all layers hold per token, from what the mixers ask of the cache manager."""
    return sum(pages.bytes_per_token(engine.dtype) for pages, _state in engine.model.cache_specs() if pages is not None)


def prefill_flops(cfg, layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d, nq, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_token = 2 * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    attention = 4 * nq * d * T * (T + 1) / 2           # causal QK^T and PV
    return layers * (per_token * T + attention) + 2 * V * H


def build_ours(cfg, layers, batch_cap, dtype, tokens_per_request=CONTEXT + 256, pages=None, page_size=None, model=None):
    import torch

    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.engine.generate import GenerationEngine
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.ops import build_library
    from llm_pipeline_b200.weights import random_tensors

    build_library()
    page_size = page_size or PAGE_SIZE
    config = resolve_config({**cfg, "num_hidden_layers": layers})
    if model is None:
        model = build_model(config)
        model.load(random_tensors(config, seed=0, dtype=dtype, device="cuda:0"), torch.device("cuda:0"), dtype)
    if pages is None:
        pages = batch_cap * (-(-tokens_per_request // page_size))
    engine = GenerationEngine(model, config, page_size=page_size, num_pages=pages, max_num_seqs=batch_cap,
                              max_num_batched_tokens=PREFILL_TOKENS, max_model_len=tokens_per_request)
    return engine


def random_prompts(vocab, count, length, seed):
    import torch

    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count, length), generator=gen).tolist()


def time_decode(engine, batch, steps, warmup, seed, e2e=True, contexts=None):
    """Device-timed decode steps through the step function, and wall-clock steps through
    ``GenerationEngine.step`` (host lists in and out). Returns a dict of figures. ``contexts``: the
    requests' context lengths when they are not all CONTEXT (device-timed part only)."""
    import torch

    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.ops import kernels
    from llm_pipeline_b200.sampling import SamplingConfig

    vocab = engine.model.spec.vocab_size
    if contexts is None:
        prompts = random_prompts(vocab, batch, CONTEXT - 1, seed)
    else:
        prompts = [random_prompts(vocab, 1, n - 1, seed + i)[0] for i, n in enumerate(contexts)]
    runner = engine.runner
    ids = [f"bench{seed}_{i}" for i in range(batch)]
    # fill the cache: every request gets its context less one token, in portions of up to 2,048 tokens
    for rid, prompt in zip(ids, prompts):
        for at in range(0, len(prompt), PREFILL_TOKENS):
            runner.step([StepEntry(rid, prompt[at:at + PREFILL_TOKENS], [])])
    last = [p[-1] for p in prompts]
    outs = [torch.empty(batch, dtype=torch.int32, device=engine.device) for _ in range(2)]

    # As the engine steps: the ids a step samples stay on the device, where the next step takes them from
    # (``StepEntry.device_token``); the host reads them a step late (the end-to-end figure below has that read in it).
    def one_step(k, before):
        if before is None:
            entries = [StepEntry(rid, [t], [0]) for rid, t in zip(ids, last)]
        else:
            entries = [StepEntry(rid, [0], [0], None, (before, i)) for i, rid in enumerate(ids)]
        return kernels.argmax(runner.step(entries), outs[k & 1])

    tokens = None
    for k in range(warmup):
        tokens = one_step(k, tokens)
    torch.cuda.synchronize()
    launches_before = kernels.launch_count
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(warmup, warmup + steps):
        tokens = one_step(k, tokens)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    launches = kernels.launch_count - launches_before
    h2d = runner.last_h2d_bytes
    for rid in ids:
        runner.release(rid)
    if not e2e:
        return {"ms": ms, "tok_s": batch * 1e3 / ms, "launches": launches, "h2d": h2d}

    # end to end: the public entry point, requests in as host token lists, tokens out as host ints
    greedy = SamplingConfig(temperature=0.0)
    e2e_prompts = random_prompts(vocab, batch, CONTEXT - 1, seed + 1)
    for p in e2e_prompts:
        engine.add_request(p, max_tokens=warmup + steps + 2 * batch + 16, sampling=greedy, ignore_eos=True)
    while any(r.num_pending > 1 or not r.output for r in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()                            # prompts, portion by portion
    for _ in range(8):
        engine.step()                            # set-up: the first decode steps of a shape run eagerly, then are captured
    for _ in range(warmup):
        engine.step()                            # the untimed warm-up steps
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    e2e_h2d = runner.last_h2d_bytes
    while engine.has_unfinished():
        engine.step()
    return {"ms": ms, "tok_s": batch * 1e3 / ms, "launches": launches, "h2d": h2d,
            "e2e_ms": e2e_ms, "e2e_tok_s": batch * 1e3 / e2e_ms, "e2e_h2d": e2e_h2d, "e2e_d2h": batch * 4}


def time_prefill(engine, tokens, repeats, warmup):
    import torch

    from llm_pipeline_b200.engine import StepEntry

    vocab = engine.model.spec.vocab_size
    runner = engine.runner
    times = []
    for i in range(warmup + repeats):
        prompt = random_prompts(vocab, 1, tokens, 500 + i)[0]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("prefill", prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.release("prefill")
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def product_labels(cfg):
    """Names the matrix products of a step after what they are in this model (for ``ops.timing.KernelTimes``)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    qkv = q + 2 * cfg["num_key_value_heads"] * cfg["head_dim"]

    def label(name, work):
        if work is None:
            return name
        _M, N, K = work
        kind = ("product_head" if N == V else "product_gate_up" if N == 2 * I else "product_qkv" if N == qkv and K == H
                else "product_down" if N == H and K == I else "product_o" if N == H and K == q else "product_other")
        return (kind + ("+swiglu" if name.endswith("+swiglu") else "") + (" (library)" if name == "mm" else "") +
                (" (library, into the residual)" if name == "mm+residual" else ""))
    return label


def breakdown_summary(table, peak, attention_bytes=0.0, attention_flops=0.0):
    """Per class: launches, microseconds, and for the products and the attention kernels what they achieved over the
    measured peak (GB/s of the bytes they must read when the rows are few, TFLOP/s otherwise)."""
    out = {}
    total = sum(e["us"] for e in table.values())
    for label, e in table.items():
        row = {"launches": e["launches"], "us": round(e["us"], 1), "share": round(e["us"] / total, 3)}
        seconds = e["us"] * 1e-6
        if label == "decode_attention" and attention_bytes:
            e["bytes"], e["rows"] = attention_bytes, 1
        if label == "paged_attention" and attention_flops:
            e["flops"], e["rows"] = attention_flops, 1 << 20
        if e["bytes"] and e["rows"] <= 64:
            row["gbs"] = round(e["bytes"] / seconds / 1e9, 1)
            row["frac_hbm"] = round(e["bytes"] / seconds / 1e9 / peak["hbm_gbs"], 3)
        elif e["flops"]:
            row["tflops"] = round(e["flops"] / seconds / 1e12, 1)
            row["frac_bf16_burst"] = round(e["flops"] / seconds / 1e12 / peak["bf16_tflops_burst"], 3)
        out[label] = row
    return {"kernel_us": round(total, 1), "classes": out}


def breakdown_of_a_step(engine, cfg, peak, entries_of, attention_bytes=0.0, attention_flops=0.0, release=()):
    """One eager step (no graph) with events around every launch, queued behind a sleeping kernel."""
    import torch

    runner = engine.runner
    graphs, runner.use_graphs = runner.use_graphs, False
    try:
        runner.step(entries_of(0))                      # untimed: first-call set-up of every kernel of the shape
        torch.cuda.synchronize()
        from llm_pipeline_b200.ops.timing import KernelTimes
        times = KernelTimes(product_labels(cfg))
        torch.cuda._sleep(int(1.5e8))                   # some 80 ms at the SM clock: the whole step queues up behind it
        with times:
            runner.step(entries_of(1))
        torch.cuda.synchronize()
    finally:
        runner.use_graphs = graphs
        for rid in release:
            runner.release(rid)
    return breakdown_summary(times.table(), peak, attention_bytes, attention_flops)


def decode_breakdown(engine, cfg, peak, batch):
    import torch

    from llm_pipeline_b200.engine import StepEntry

    vocab = engine.model.spec.vocab_size
    prompts = random_prompts(vocab, batch, CONTEXT - 2, 77)
    ids = [f"breakdown{i}" for i in range(batch)]
    for rid, prompt in zip(ids, prompts):
        engine.runner.step([StepEntry(rid, prompt, [])])
    layers = len(engine.model.schedule)
    kv_bytes = batch * CONTEXT * kv_bytes_per_token(engine)
    out = breakdown_of_a_step(engine, cfg, peak, lambda k: [StepEntry(rid, [p[k]], [0]) for rid, p in zip(ids, prompts)],
                              attention_bytes=kv_bytes, release=ids)
    out["launches_per_step"] = sum(c["launches"] for c in out["classes"].values())
    out["layers"] = layers
    return out


def prefill_breakdown(engine, cfg, peak, tokens):
    from llm_pipeline_b200.engine import StepEntry

    vocab = engine.model.spec.vocab_size
    prompts = random_prompts(vocab, 2, tokens, 88)
    layers = len(engine.model.schedule)
    flops = layers * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    runner = engine.runner

    def entries(k):
        if k:
            runner.release("prefill_breakdown")
        return [StepEntry("prefill_breakdown", prompts[k], [tokens - 1])]

    return breakdown_of_a_step(engine, cfg, peak, entries, attention_flops=flops, release=["prefill_breakdown"])


def plain_baseline(cfg, layers, tokens):
    """This repository's plain PyTorch implementation (tests/plain_qwen3.py: whole sequences, no cache, library
    products) in bfloat16 on the GPU with the same seeded weights: the time of one forward over ``tokens`` tokens, which
    is its prefill and, having no cache, also what one more decoded token costs it at that context."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3 as plain

    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.weights import random_tensors

    config_json = {**cfg, "num_hidden_layers": layers}
    source = random_tensors(resolve_config(config_json), seed=0, dtype=torch.bfloat16, device="cuda:0")
    weights = {name: source.get(name) for name in source.names()}
    ids = random_prompts(cfg["vocab_size"], 1, tokens, 99)[0]
    times = []
    with torch.no_grad():
        for i in range(5):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            logits = plain.forward_logits(config_json, weights, ids, dtype=torch.bfloat16, rows=[tokens - 1])
            token = int(logits[0].argmax())
            stop.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(start.elapsed_time(stop))
    del weights, logits
    torch.cuda.empty_cache()
    ms = sorted(times)[len(times) // 2]
    return {"what": "tests/plain_qwen3.py, bfloat16, whole sequence per token (no cache)", "context": tokens, "layers": layers,
            "ms_per_forward": round(ms, 3), "decode_b1": round(1e3 / ms, 2), "prefill": round(tokens * 1e3 / ms, 1), "last_token": token}


def selfcheck(cfg, batches=(8, 64), prompt_tokens=48, new_tokens=4):
    """Outside every timed region: a two-layer model of the benchmark's widths generates greedily through the Python
    entry point in steps of 8 and of 64 requests (the fused streaming products, the library products and both decode
    attention streams), and every generated token must be the plain implementation's greedy choice at its place, or
    lose to it by less than the bfloat16 rounding noise of these logits (0.25 on logits that reach 7)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3 as plain

    from llm_pipeline_b200.weights import random_tensors

    torch.backends.cuda.matmul.allow_tf32 = False
    engine = build_ours(cfg, 2, max(batches), torch.bfloat16, tokens_per_request=256)
    config_json = {**cfg, "num_hidden_layers": 2}
    source = random_tensors(engine.config, seed=0, dtype=torch.bfloat16, device="cuda:0")
    weights = {name: source.get(name).float() for name in source.names()}
    report = {}
    for batch in batches:
        prompts = random_prompts(cfg["vocab_size"], batch, prompt_tokens, 4000 + batch)
        results = engine.generate(prompts, max_tokens=new_tokens, temperature=0.0, ignore_eos=True)
        equal = close = wrong = 0
        for prompt, result in zip(prompts, results):
            ids = list(prompt) + list(result.token_ids)
            rows = list(range(len(prompt) - 1, len(ids) - 1))
            logits = plain.forward_logits(config_json, weights, ids, rows=rows)
            for row, token in zip(logits, result.token_ids):
                best = int(row.argmax())
                if best == token:
                    equal += 1
                elif float(row[best] - row[token]) < 0.25:
                    close += 1
                else:
                    wrong += 1
        report[f"batch_{batch}"] = {"tokens": batch * new_tokens, "equal": equal, "within_rounding": close, "wrong": wrong}
    del engine, weights
    torch.cuda.empty_cache()
    report["ok"] = all(r["wrong"] == 0 and r["equal"] >= 0.9 * r["tokens"] for r in report.values() if isinstance(r, dict))
    return report


def mix_workload(cfg, layers):
    """A continuous-batching mix through the Python entry point: 64 requests with prompt lengths uniform in
    [16, 2048] and 128 decoded tokens each (seeded), context up to 4,096; returns its figures."""
    import torch

    from llm_pipeline_b200.sampling import SamplingConfig

    engine = build_ours(cfg, layers, 64, torch.bfloat16, tokens_per_request=2048 + 128 + 16)
    gen = torch.Generator().manual_seed(7)
    lengths = torch.randint(16, 2049, (64,), generator=gen).tolist()
    prompts = [random_prompts(cfg["vocab_size"], 1, n, 1000 + i)[0] for i, n in enumerate(lengths)]
    greedy = SamplingConfig(temperature=0.0)
    warm = engine.generate([prompts[0][:64]], max_tokens=4, temperature=0.0)      # builds kernels' first-call state
    del warm
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        engine.add_request(p, max_tokens=128, sampling=greedy, ignore_eos=True)
    steps = 0
    while engine.has_unfinished():
        engine.step()
        steps += 1
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    total = sum(lengths) + 64 * 128
    stats = engine.stats()
    del engine
    torch.cuda.empty_cache()
    return {"requests": 64, "prompt_tokens": sum(lengths), "decoded_tokens": 64 * 128, "seconds": round(seconds, 3),
            "tokens_per_s": round(total / seconds, 1), "decoded_tokens_per_s": round(64 * 128 / seconds, 1), "steps": steps,
            "mean_step_ms": round(seconds * 1e3 / steps, 3), "preemptions": stats["preemptions"]}


def run_mix(args):
    name, cfg = SHAPES[args.shape]
    layers = args.layers or cfg["num_hidden_layers"]
    print(json.dumps({"workload": "mix", "model": name, "layers": layers, **mix_workload(cfg, layers)}))
    return 0


def further_points(args):
    """Other sizes through the same engine, each at its full depth: the Qwen3-0.6B shape under the continuous-batching
    mix (total tokens per second through the Python entry point), and decode at batch 8 and 2,048 tokens of context
    at the Qwen3-32B shape (65 GB of weights)."""
    import torch

    out = {}
    _name, small = SHAPES["0.6b"]
    out["qwen3_0.6b_mix_64_requests"] = mix_workload(small, small["num_hidden_layers"])["tokens_per_s"]
    _name, large = SHAPES["32b"]
    engine = build_ours(large, large["num_hidden_layers"], 8, torch.bfloat16)
    r = time_decode(engine, 8, 8, args.warmup, seed=40, e2e=False)
    out["qwen3_32b_decode_b8"] = round(r["tok_s"], 1)
    step_bytes = weight_bytes(large, large["num_hidden_layers"]) + 8 * (CONTEXT + args.warmup + 4) * kv_bytes_per_token(engine)
    out["qwen3_32b_decode_b8_gbs"] = round(step_bytes / (r["ms"] * 1e-3) / 1e9, 1)
    del engine
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch

    if args.workload == "mix":
        return run_mix(args)
    name, cfg = SHAPES[args.shape]
    layers = args.layers or cfg["num_hidden_layers"]
    peak = peaks()
    dtype = torch.bfloat16
    # room per request: the context, the set-up, warm-up and timed decode steps, in whole pages
    room = -(-(CONTEXT + 64 + args.warmup + args.steps) // 256) * 256
    contexts = [int(n) for n in args.contexts.split(",")] if args.contexts else None
    if contexts:
        if args.only != "decode":
            print("--contexts goes with --only decode")
            return 2
        args.batch = len(contexts)
        longest = -(-(max(contexts) + 64 + args.warmup + args.steps) // 256) * 256
        pages = sum(-(-(n + 64 + args.warmup + args.steps) // PAGE_SIZE) for n in contexts)
        engine = build_ours(cfg, layers, args.batch, dtype, tokens_per_request=longest, pages=pages)
    else:
        engine = build_ours(cfg, layers, max(64, args.batch), dtype, tokens_per_request=max(CONTEXT + 256, room))
    clocks = ClockSampler()
    clocks.start()
    if args.only == "prefill":
        clocks.stop()
        prefill_ms = time_prefill(engine, PREFILL_TOKENS, repeats=2, warmup=3)
        print(json.dumps({"only": "prefill", "layers": layers, "prefill_ms": round(prefill_ms, 3)}))
        return 0
    main = time_decode(engine, args.batch, args.steps, args.warmup, seed=1, e2e=args.only == "all", contexts=contexts)
    clock_info = clocks.stop()
    if args.only == "decode":
        line = {"only": "decode", "layers": layers, "batch": args.batch, "ms_per_step": round(main["ms"], 4)}
        if contexts:
            line["contexts"] = args.contexts
        print(json.dumps(line))
        return 0
    points = {}
    for b in (1, 64):
        r = time_decode(engine, b, max(5, args.steps // 2), args.warmup, seed=10 + b, e2e=False)
        points[f"decode_b{b}"] = round(r["tok_s"], 1)
    prefill_ms = time_prefill(engine, PREFILL_TOKENS, repeats=5, warmup=3)
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    kv_per_token = kv_bytes_per_token(engine)
    breakdown = baselines = check = None
    if not args.lean:
        breakdown = {f"decode_b{args.batch}": decode_breakdown(engine, cfg, peak, args.batch),
                     f"prefill_{PREFILL_TOKENS}": prefill_breakdown(engine, cfg, peak, PREFILL_TOKENS)}
        # the same batch with pages of 32 tokens (half as many TMA boxes in the decode attention stream)
        other_page = 32 if PAGE_SIZE != 32 else 16
        wide = build_ours(cfg, layers, max(64, args.batch), dtype, tokens_per_request=max(CONTEXT + 256, room), page_size=other_page,
                          model=engine.model)
        r = time_decode(wide, args.batch, max(5, args.steps // 2), args.warmup, seed=30, e2e=False)
        points[f"decode_b{args.batch}_page{other_page}"] = round(r["tok_s"], 1)
        del wide
        del engine
        torch.cuda.empty_cache()
        baselines = {"plain_pytorch": plain_baseline(cfg, layers, CONTEXT)}
        check = selfcheck(cfg)
        if args.shape == "8b" and not args.layers:
            points.update(further_points(args))
    step_bytes = weight_bytes(cfg, layers) + args.batch * (CONTEXT + args.warmup + args.steps // 2) * kv_per_token
    achieved = step_bytes / (main["ms"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch}, 2,048-token context ({name.split()[0]} bf16)",
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "impl": "ours",
        "config": {"model": name, "layers": layers, "layers_of_model": cfg["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "page_size": PAGE_SIZE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2, no flush", "peaks": peak["source"]},
        "e2e": {"value": round(main["e2e_tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(main["e2e_ms"], 4),
                "h2d_bytes_per_step": main["e2e_h2d"], "d2h_bytes_per_step": main["e2e_d2h"]},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
                    "frac_burst": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops_burst"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_info,
    }
    if breakdown is not None:
        line["breakdown"] = breakdown
        line["baselines"] = baselines
        line["selfcheck"] = check
    print(json.dumps(line))
    return 0 if check is None or check["ok"] else 1


def run_reference(args):
    """The reference's own model class and cache loop, unmodified, from baseline/_ref."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "llm_pipeline")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --no-deps --target)"}))
        return 0
    sys.path.insert(0, ref_root)
    try:
        import torch
        from llm_pipeline.models.qwen3.custom_builder import Qwen3Config as RefConfig, Qwen3ForCausalLM
    except Exception as e:      # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:200]}))
        return 0
    cfg = dict(QWEN3_8B)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    torch.manual_seed(0)
    with torch.device("cuda:0"):
        torch.set_default_dtype(torch.bfloat16)
        model = Qwen3ForCausalLM(RefConfig(**cfg)).eval()
        torch.set_default_dtype(torch.float32)
    for p in model.parameters():
        p.data.normal_(0, 0.02)
    batch = args.batch
    ids = torch.tensor(random_prompts(cfg["vocab_size"], batch, CONTEXT - 1, 1), device="cuda:0")
    clocks = ClockSampler()
    with torch.no_grad():
        out = model(input_ids=ids, use_cache=True)
        past = out.past_key_values
        token = out.logits[:, -1, :].argmax(-1, keepdim=True)

        def one_step(token, past):
            out = model(input_ids=token, past_key_values=past, use_cache=True)
            nxt = out.logits[:, -1, :].argmax(-1, keepdim=True)
            return torch.tensor(nxt.tolist(), device="cuda:0"), out.past_key_values

        for _ in range(args.warmup):
            token, past = one_step(token, past)
        torch.cuda.synchronize()
        clocks.start()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        for _ in range(args.steps):
            token, past = one_step(token, past)
        stop.record()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    ms = start.elapsed_time(stop) / args.steps
    line = {
        "metric": "decode tok/s at batch 8, 2,048-token context (Qwen3-8B bf16)", "impl": "reference",
        "value": round(batch * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_of_model": QWEN3_8B["num_hidden_layers"],
                   "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
                   "path": "Qwen3ForCausalLM.forward with past_key_values"},
        "e2e": {"value": round(batch * 1e3 / wall_ms, 1), "unit": "tokens/s", "h2d_bytes_per_step": batch * 8,
                "d2h_bytes_per_step": batch * 8},
        "gpu_launches": 0, "clocks": clocks.stop(),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference", "plain"),
                        help="plain: this repository's plain PyTorch implementation (tests/plain_qwen3.py) alone")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--shape", default="8b", choices=tuple(SHAPES), help="layer sizes (default: Qwen3-8B)")
    parser.add_argument("--workload", default="decode", choices=("decode", "mix"),
                        help="mix: the continuous-batching mix of 64 requests through the Python entry point")
    parser.add_argument("--contexts", default="", help="with --only decode: the requests' context lengths, comma-separated "
                        "(a batch of uneven lengths), instead of --batch requests of 2,048 tokens")
    parser.add_argument("--only", default="all", choices=("all", "decode", "prefill"),
                        help="run one part only (for profiler captures on a small case); the line then lacks the other parts")
    parser.add_argument("--lean", action="store_true", help="leave out the per-kernel breakdown, the page-size point, the plain "
                        "PyTorch baseline and the self-check")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per page of the key/value cache")
    args = parser.parse_args()
    globals()["PAGE_SIZE"] = args.page_size
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("bench.py measures a single-GPU engine: run it with --gpus 1 (no multi-GPU path is built)")
        return 2
    args.warmup = max(3, args.warmup)
    if args.impl == "plain":
        name, cfg = SHAPES[args.shape]
        out = plain_baseline(cfg, args.layers or cfg["num_hidden_layers"], CONTEXT)
        print(json.dumps({"impl": "plain", "metric": f"decode tok/s at batch 1, 2,048-token context ({name.split()[0]} bf16)",
                          "value": out["decode_b1"], "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", **out}))
        return 0
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
