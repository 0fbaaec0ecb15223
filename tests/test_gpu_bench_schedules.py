"""Decode steps of the sizes the benchmark times, at the widths and the vocabulary of Qwen3-8B.

Two layers with hidden 4096, 32 query and 8 key/value heads of 128, intermediate 12288 and the real vocabulary of
151,936: the shapes every fast kernel of a decode step is tuned for. Steps of 5, 8, 9, 16, 17, 32 and 64 live
requests with contexts that cross page edges, 128-key edges and 2,048 keys are compared with the plain
implementation, run on the GPU in float64 so that the oracle's own rounding does not count. The tests also say
which product and which decode-attention kernel each step size took, since the choice follows the step's shape,
and pin how far a request's logits may depend on who else is in the step.
"""

import contextlib

import pytest
import torch

import helpers as H
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

VOCAB = 151936
CONFIG = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 4096,
          "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
          "vocab_size": VOCAB, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
          "max_position_embeddings": 4096}
BATCHES = (5, 8, 9, 16, 17, 32, 64)
STEPS_PER_BATCH = 3                      # the first step of a shape runs eagerly, the second is captured, the third replays
PAGE = 16
PEAK = 2.0                               # factor on the second layer's q/k norm weights: scores of spread 4 instead of 1
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def context_lengths():
    """64 contexts: the first ones placed so that their decoded tokens cross 2,048 keys, a 128-key edge, a page edge and
    1,024 keys, one that starts from a single token, then seeded lengths up to 400."""
    fixed = [2040, 120, 10, 255, 1, 500, 1015, 640]
    gen = torch.Generator().manual_seed(11)
    return fixed + torch.randint(1, 401, (64 - len(fixed),), generator=gen).tolist()


def decode_tokens_of(i: int) -> int:
    return STEPS_PER_BATCH * sum(1 for b in BATCHES if b > i)


@pytest.fixture(scope="module")
def case():
    """Weights (bfloat16 values held in float32 and in float64 on the GPU; the second layer's q/k norm weights are
    doubled, which makes its softmax peaked: a few keys among hundreds carry the output, so a key that a kernel
    drops or reads from the wrong page shows in the logits), the requests' tokens, the oracle's logits, and as a
    yardstick how far the plain implementation itself is from the oracle when it runs in float32 and in bfloat16."""
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.weights import random_tensors
    torch.backends.cuda.matmul.allow_tf32 = False
    config = resolve_config(CONFIG)
    source = random_tensors(config, seed=5, dtype=torch.bfloat16, device="cuda:0")
    weights = {name: source.get(name).float() for name in source.names()}
    for name in ("model.layers.1.self_attn.q_norm.weight", "model.layers.1.self_attn.k_norm.weight"):
        weights[name] = (weights[name] * PEAK).to(torch.bfloat16).float()
    w64 = {name: t.double() for name, t in weights.items()}
    contexts = context_lengths()
    tokens = [H.random_tokens(VOCAB, n + decode_tokens_of(i), 7000 + i) for i, n in enumerate(contexts)]
    want = []
    for i, n in enumerate(contexts):
        rows = list(range(n, n + decode_tokens_of(i)))
        want.append(plain.forward_logits(CONFIG, w64, tokens[i], dtype=torch.float64, rows=rows).float().cpu())
    del w64
    yardstick = {}
    for dtype in (torch.float32, torch.bfloat16):
        w = {name: t.to(dtype) for name, t in weights.items()}
        worst, square, count = 0.0, 0.0, 0
        for i in (0, 1, 3, 6, 20):
            rows = list(range(contexts[i], contexts[i] + decode_tokens_of(i)))
            diff = plain.forward_logits(CONFIG, w, tokens[i], dtype=dtype, rows=rows).float().cpu() - want[i]
            worst, square, count = max(worst, float(diff.abs().max())), square + float(diff.pow(2).sum()), count + diff.numel()
        yardstick[dtype] = (worst, (square / count) ** 0.5)
        del w
    torch.cuda.empty_cache()
    return {"config": config, "weights": weights, "contexts": contexts, "tokens": tokens, "want": want, "yardstick": yardstick}


def runner_for(case, dtype, num_pages=2048, max_requests=64):
    from llm_pipeline_b200.cache import CacheManager
    from llm_pipeline_b200.engine import ModelRunner
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.weights import DictSource
    model = build_model(case["config"]).load(DictSource(case["weights"]), torch.device("cuda:0"), dtype)
    cache = CacheManager(model.cache_specs(), page_size=PAGE, num_pages=num_pages, max_requests=max_requests,
                         max_request_tokens=4096, device=model.device, dtype=dtype)
    return ModelRunner(model, cache)


@contextlib.contextmanager
def recorded_kernels(log):
    """Every call of a product or decode-attention entry point goes into ``log`` as (name, rows of x or of the step,
    weight rows or None, uneven or None) while the block runs."""
    from llm_pipeline_b200.ops import kernels
    names = ("gemm_stream", "gemm_stream_fused", "gemm_stream_swiglu", "gemm_stream_tc", "gemm_tc", "gemm_skinny",
             "gemm_simt", "decode_attention", "gemm_stream_chain")
    saved = {name: getattr(kernels, name) for name in names}
    library_mm = torch.mm

    def wrap(name, fn):
        def call(*args, **kwargs):
            if name == "decode_attention":
                log.append((name, args[2].shape[0], None, bool(kwargs.get("uneven", False))))
            elif name == "gemm_stream_chain":
                log.append((name, args[1], len(args[0]), None))          # rows, phases
            else:
                log.append((name, args[0].shape[0], args[1].shape[0], None))
            return fn(*args, **kwargs)
        return call

    def mm(a, b, **kwargs):
        log.append(("library", a.shape[0], b.shape[1], None))
        return library_mm(a, b, **kwargs)

    for name in names:
        setattr(kernels, name, wrap(name, saved[name]))
    torch.mm = mm
    try:
        yield
    finally:
        for name in names:
            setattr(kernels, name, saved[name])
        torch.mm = library_mm


def prefill(runner, rid, tokens, portion=2048):
    from llm_pipeline_b200.engine import StepEntry
    for at in range(0, len(tokens), portion):
        runner.step([StepEntry(rid, tokens[at:at + portion], [])])


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_steps_of_the_benchmark_sizes(case, dtype):
    from llm_pipeline_b200.engine import StepEntry
    runner = runner_for(case, dtype)
    contexts, tokens, want = case["contexts"], case["tokens"], case["want"]
    for i, n in enumerate(contexts):
        prefill(runner, i, tokens[i][:n])
    done = [0] * 64
    scale = max(float(w.abs().max()) for w in want)
    # float32: 1e-4 absolute on logits that reach about 7 here, against an oracle in float64 (the plain implementation
    # in float32 is itself 6e-5 from it). bfloat16: rounding to 8 bits of mantissa at the input of every matrix product
    # of K = 4,096 and 12,288 is worth 1 to 2 % of the largest logit at these widths; the bound is the yardstick: the
    # engine is nowhere further from the oracle than the plain implementation run in bfloat16 is at its worst place,
    # and on average (root mean square of each step) closer than that implementation is on average.
    yard_worst, yard_rms = case["yardstick"][dtype]
    tol = 1e-4 if dtype == torch.float32 else yard_worst
    worst = 0.0
    paths = {}
    for batch in BATCHES:
        for s in range(STEPS_PER_BATCH):
            log = []
            with recorded_kernels(log):
                logits = runner.step([StepEntry(i, [tokens[i][contexts[i] + done[i]]], [0]) for i in range(batch)])
            if s == 0:
                paths[batch] = log
            got = logits.float().cpu()
            if dtype == torch.bfloat16:
                rms = float(torch.cat([got[i] - want[i][done[i]] for i in range(batch)]).pow(2).mean().sqrt())
                assert rms <= yard_rms, f"step {s} of batch {batch}: root mean square difference {rms:.3e} > {yard_rms:.3e}"
            for i in range(batch):
                diff = float((got[i] - want[i][done[i]]).abs().max())
                assert diff <= tol, f"{dtype}: step {s} of batch {batch}, request {i} (context {contexts[i] + done[i]}): {diff:.3e} > {tol:.1e}"
                worst = max(worst, diff)
                if dtype == torch.bfloat16 and float(torch.topk(want[i][done[i]], 2).values.diff().abs()) > 4 * tol:
                    assert int(got[i].argmax()) == int(want[i][done[i]].argmax())
                done[i] += 1
    print(f"\n{dtype}: largest logit {scale:.3f}, largest difference over all decode steps {worst:.3e} "
          f"(plain implementation in this type: {yard_worst:.3e})")
    if dtype == torch.bfloat16:
        # every size replays its graph, but for the one step in which the longest request's block table passes 128 pages
        # (2,048 keys): a wider table is another graph, whose first step runs eagerly again
        assert runner.graph_replays >= len(BATCHES) * (STEPS_PER_BATCH - 1) - 1
    runner.cache.check()
    # which kernels the eager first step of every size took
    for batch, log in paths.items():
        names = {entry[0] for entry in log}
        if dtype == torch.float32:
            assert names == {"gemm_simt", "decode_attention"}, (batch, names)
            continue
        if batch <= 8:
            assert "gemm_stream_fused" in names and "library" not in names, (batch, names)
        elif batch <= 16:
            assert ("gemm_stream", batch, 4096, None) in log, (batch, log)              # the narrow products stream
            assert ("library", batch, 24576, None) in log, (batch, log)                 # the wide ones do not
        if 8 < batch <= 32:
            assert ("gemm_stream_tc", batch, VOCAB, None) in log, (batch, log)          # the head on tcgen05
        if batch > 32:
            assert names <= {"library", "decode_attention"}, (batch, names)
        uneven = [entry[3] for entry in log if entry[0] == "decode_attention"]
        assert len(uneven) == 2 and uneven[0] == uneven[1]
        if batch == 64:
            assert uneven[0], "64 requests of 8 key/value heads are more than two row groups per SM: the list kernel"


def decode_alone_and_in_company(case, dtype, runner, company, place, portions=None, steps=4):
    """Logits [steps, vocab] of one request (300 tokens of context, then ``steps`` decoded tokens) that decodes at row
    ``place`` of steps shared with ``company`` other requests."""
    from llm_pipeline_b200.engine import StepEntry
    contexts, tokens = case["contexts"], case["tokens"]
    mine = H.random_tokens(VOCAB, 300 + steps, 4242)
    others = list(range(1, 1 + company))
    their_next = {i: H.random_tokens(VOCAB, steps, 9000 + i) for i in others}
    for i in others:
        prefill(runner, i, tokens[i][:contexts[i]])
    if portions is None:
        prefill(runner, "x", mine[:300])
    else:
        at, k = 0, 0
        while at < 300:
            n = min(portions[k % len(portions)], 300 - at)
            runner.step([StepEntry("x", mine[at:at + n], [])])
            at, k = at + n, k + 1
    out = []
    for s in range(steps):
        entries = [StepEntry(i, [their_next[i][s]], []) for i in others]
        entries.insert(min(place, len(entries)), StepEntry("x", [mine[300 + s]], [0]))
        out.append(runner.step(entries)[0].clone())
    for rid in others + ["x"]:
        runner.release(rid)
    return torch.stack(out), mine


@pytest.mark.parametrize("dtype", DTYPES)
def test_logits_do_not_depend_on_the_company(case, dtype):
    """The same request decoded alone, beside 3 others and beside 63 others, and after a prompt cut into portions.
    float32: the same bits (every kernel of that path works on a row with operations that depend on the row alone:
    fixed 128-key ranges in decode attention, a fixed order along K in the products). bfloat16: the products and the
    decode-attention kernels follow the step's shape (streaming product, tcgen05 head, library; one of two decode
    streams, whose blocks per row group follow the number of requests), so sums meet in another order; the bound
    below is what that may cost."""
    runner = runner_for(case, dtype)
    alone, mine = decode_alone_and_in_company(case, dtype, runner, 0, 0)
    with_3, _ = decode_alone_and_in_company(case, dtype, runner, 3, 2)
    with_63, _ = decode_alone_and_in_company(case, dtype, runner, 63, 40)
    cut, _ = decode_alone_and_in_company(case, dtype, runner, 0, 0, portions=(37, 2, 64, 5, 128))
    runner.cache.check()
    if dtype == torch.float32:
        assert torch.equal(alone, with_3), float((alone - with_3).abs().max())
        assert torch.equal(alone, with_63), float((alone - with_63).abs().max())
        assert torch.equal(alone, cut), float((alone - cut).abs().max())
        return
    # Up to 8 rows every product is the streaming kernel, whose order along K does not depend on the rows: the same bits.
    assert torch.equal(alone, with_3), float((alone - with_3).abs().max())
    # Beyond that another product kernel adds along K in another order. One differing bit in a float32 sum flips the
    # rounding to bfloat16 of some activation, and from there on the step is another draw of the same rounding noise
    # that separates the engine from the oracle. So the bound is that noise: no further from "alone" than "alone" is
    # from the oracle at its worst place, and on average no more than two independent draws differ (sqrt 2, with slack 1.5).
    w64 = {name: t.double() for name, t in case["weights"].items()}
    oracle = plain.forward_logits(CONFIG, w64, mine, dtype=torch.float64, rows=list(range(300, len(mine)))).float()
    del w64
    noise = alone.float() - oracle
    largest = float(alone.abs().max())
    for name, other in (("beside 63 others", with_63), ("prompt in portions", cut)):
        diff = (alone - other).float()
        print(f"\nbfloat16, {name}: largest difference {float(diff.abs().max()):.3e}, root mean square {float(diff.pow(2).mean().sqrt()):.3e}; "
              f"alone against the oracle {float(noise.abs().max()):.3e} and {float(noise.pow(2).mean().sqrt()):.3e}; largest logit {largest:.2f}")
        assert float(diff.abs().max()) <= float(noise.abs().max()), name
        assert float(diff.pow(2).mean().sqrt()) <= 1.5 * float(noise.pow(2).mean().sqrt()), name


def test_products_of_a_decode_step_as_one_chain_give_the_same_bits(case, monkeypatch):
    """The optional path that runs the products between two attentions as phases of one persistent launch
    (``ops.linear.CHAIN``): the same logits, bit for bit, as the products launched one by one, eagerly and replayed."""
    from llm_pipeline_b200.engine import StepEntry
    import importlib
    linear = importlib.import_module("llm_pipeline_b200.ops.linear")      # (the package also exports the function of that name)
    contexts, tokens = case["contexts"], case["tokens"]
    got = {}
    for chained in (False, True):
        monkeypatch.setattr(linear, "CHAIN", chained)
        runner = runner_for(case, torch.bfloat16, num_pages=512, max_requests=8)
        for i in range(1, 8):
            prefill(runner, i, tokens[i][:contexts[i]])
        rows, log = [], []
        with recorded_kernels(log):
            for s in range(3):
                rows.append(runner.step([StepEntry(i, [tokens[i][contexts[i] + s]], [0]) for i in range(1, 8)]).clone())
        got[chained] = torch.stack(rows)
        chains = [entry for entry in log if entry[0] == "gemm_stream_chain"]
        assert (len(chains) > 0) == chained
        if chained:
            assert ("gemm_stream_chain", 7, 4, None) in log and ("gemm_stream_chain", 7, 3, None) in log     # the last layer's: three
        del runner
    assert torch.equal(got[False], got[True])
