"""Generation through the entry points, and trace replay as a program."""

import json
import os
import subprocess
import sys

import pytest
import torch

import helpers as H
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def engine_for(folder, dtype, **kw):
    from llm_pipeline_b200.inference import Qwen3InferenceConfig, Qwen3InferenceEngine
    defaults = dict(model_path=folder, dtype=dtype, block_size=8, num_blocks=128, max_sequence_length=512,
                    max_batch_size=8, max_num_batched_tokens=64)
    defaults.update(kw)
    return Qwen3InferenceEngine(Qwen3InferenceConfig(**defaults))


def clear_choices(config, weights, prompt, generated, margin):
    """How many of the first greedy choices of the plain implementation win by more than ``margin`` (up to the first
    that does not: after a near tie the two sequences may part for good)."""
    ids = list(prompt)
    for n, token in enumerate(generated):
        logits = plain.forward_logits(config, weights, ids)[-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) <= margin:
            return n
        ids.append(token)
    return len(generated)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tiny,seed", [(plain.TINY_A, 0), (plain.TINY_B, 1)], ids=["a", "b"])
def test_greedy_generation_matches_plain(tmp_path, tiny, seed, dtype):
    folder, weights = H.make_case(tmp_path, tiny, seed, dtype, std=0.08)
    engine = engine_for(folder, dtype)
    prompts = [H.random_tokens(tiny["vocab_size"], n, 300 + n) for n in (1, 9, 24, 40)]   # 1: the first token of a sequence
    got = engine.generate(prompts, max_tokens=8, temperature=0.0)
    checked, prompts_checked = 0, 0
    for prompt, tokens in zip(prompts, got):
        want = plain.greedy_generate(tiny, weights, prompt, 8)
        # float32: every token; bfloat16: every token up to the first whose plain choice wins by less than 0.05
        n = len(want) if dtype == torch.float32 else clear_choices(tiny, weights, prompt, want, 0.05)
        assert tokens[:n] == want[:n], (len(prompt), n, tokens, want)
        checked += n
        prompts_checked += n > 0
    assert checked >= (32 if dtype == torch.float32 else 16) and prompts_checked >= 3, (checked, prompts_checked)
    single = engine.generate(prompts[2], max_tokens=8, temperature=0.0)
    assert single == got[2]
    assert engine.engine.cache.num_live == 0


def test_long_decoding_stays_exact(tmp_path):
    folder, weights = H.make_case(tmp_path, plain.TINY_A, 0, torch.float32, std=0.08)
    engine = engine_for(folder, torch.float32, block_size=16)
    prompt = H.random_tokens(256, 5, 42)
    tokens = engine.generate(prompt, max_tokens=150, temperature=0.0)
    assert len(tokens) == 150
    logits = plain.forward_logits(plain.TINY_A, weights, prompt + tokens[:-1])
    assert logits[4:].argmax(dim=-1).tolist() == tokens      # every decoded token is the plain argmax at its place


def test_sampling_is_seeded_and_independent_of_the_batch(tmp_path):
    from llm_pipeline_b200.sampling import uniform_of
    tiny = plain.TINY_B
    folder, weights = H.make_case(tmp_path, tiny, 1, torch.float32, std=0.08)
    engine = engine_for(folder, torch.float32)
    prompts = [H.random_tokens(tiny["vocab_size"], n, 500 + n) for n in (1, 9, 24, 40)]
    a = engine.generate(prompts, max_tokens=6, temperature=0.7, top_k=0, top_p=1.0, seed=123)
    b = engine.generate(prompts, max_tokens=6, temperature=0.7, top_k=0, top_p=1.0, seed=123)
    assert a == b
    alone = engine.generate([prompts[2]], max_tokens=6, temperature=0.7, top_k=0, top_p=1.0, seed=125)
    assert alone[0] == a[2]                                  # prompt i draws with seed + i, whoever else is in the batch
    other = engine.generate(prompts, max_tokens=6, temperature=0.7, top_k=0, top_p=1.0, seed=7)
    assert other != a
    # every draw is the inverse-CDF pick of the plain sampler for the same uniform number
    for i, (prompt, tokens) in enumerate(zip(prompts, a)):
        ids = list(prompt)
        for step, token in enumerate(tokens):
            probs = plain.filtered_probs(plain.forward_logits(tiny, weights, ids)[-1], 0.7)
            cdf = torch.cumsum(probs.double(), 0)
            u = uniform_of(123 + i, step)
            assert float(cdf[token] - probs[token].double()) - 1e-4 <= u <= float(cdf[token]) + 1e-4
            ids.append(token)
    filtered = engine.generate(prompts, max_tokens=6, temperature=0.7, top_k=5, top_p=0.9, seed=3)
    for prompt, tokens in zip(prompts, filtered):
        ids = list(prompt)
        for token in tokens:
            probs = plain.filtered_probs(plain.forward_logits(tiny, weights, ids)[-1], 0.7, top_k=5, top_p=0.9)
            assert probs[token] > 0
            ids.append(token)


def test_preemption_recomputes_to_the_same_tokens(tmp_path):
    tiny = plain.TINY_A
    folder, weights = H.make_case(tmp_path, tiny, 0, torch.float32, std=0.08)
    prompts = [H.random_tokens(tiny["vocab_size"], n, 700 + n) for n in (20, 18, 22)]
    roomy = engine_for(folder, torch.float32, block_size=4, num_blocks=256)
    want = roomy.generate(prompts, max_tokens=24, temperature=0.0)
    tight = engine_for(folder, torch.float32, block_size=4, num_blocks=26)    # 104 token slots for 3 x (up to 46)
    results = tight.generate_ids(prompts, max_tokens=24, temperature=0.0)
    assert [r.token_ids for r in results] == want
    assert sum(r.preemptions for r in results) >= 1 and tight.engine.scheduler.num_preemptions >= 1
    assert tight.engine.cache.num_live == 0 and tight.engine.cache.groups[0].pool.num_free == 26
    assert tight.engine.cache.pages_reused > 0


def test_eos_and_stats(tmp_path):
    tiny = plain.TINY_A
    folder, weights = H.make_case(tmp_path, tiny, 0, torch.float32, std=0.08)
    prompt = H.random_tokens(256, 7, 9)
    free_run = plain.greedy_generate(tiny, weights, prompt, 12)
    engine = engine_for(folder, torch.float32, eos_token_id=free_run[4])
    out = engine.generate_ids([prompt], max_tokens=12, temperature=0.0)[0]
    stop_at = free_run.index(free_run[4])
    assert out.token_ids == free_run[:stop_at + 1] and out.finish_reason == "stop"
    stats = engine.get_stats()
    assert stats["finished"] == 1 and stats["tokens_prefilled"] == 7 and stats["live_requests"] == 0


def test_streaming_and_cleanup(tmp_path):
    tiny = plain.TINY_A
    folder, weights = H.make_case(tmp_path, tiny, 0, torch.float32, std=0.08)
    engine = engine_for(folder, torch.float32)
    prompt = H.random_tokens(256, 9, 77)
    streamed = list(engine.stream_generate(prompt, max_tokens=7, temperature=0.0))
    assert streamed == plain.greedy_generate(tiny, weights, prompt, 7)
    assert engine.continuous_batch_generate([prompt], max_tokens=7, temperature=0.0) == [streamed]
    engine.engine.add_request(prompt, max_tokens=50)
    engine.engine.step()
    assert engine.engine.cache.num_live == 1
    engine.cleanup()
    assert engine.engine.cache.num_live == 0 and not engine.engine.has_unfinished()


def test_real_layer_widths_two_layers():
    """Two layers with the widths of Qwen3-8B (hidden 4096, 32 query and 8 key/value heads of 128,
    intermediate 12288) and a vocabulary that is no multiple of anything: the sizes the fast kernels are
    tuned for, against the plain implementation run on the GPU in float32 (TF32 off)."""
    from llm_pipeline_b200.cache import CacheManager
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.engine import ModelRunner
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.weights import DictSource, random_tensors
    torch.backends.cuda.matmul.allow_tf32 = False
    config_json = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 4096,
                   "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
                   "vocab_size": 10007, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
                   "max_position_embeddings": 4096}
    config = resolve_config(config_json)
    source = random_tensors(config, seed=5, dtype=torch.bfloat16, device="cuda:0")
    weights = {name: source.get(name).float() for name in source.names()}       # bfloat16 values, held in float32
    requests = {"p": H.random_tokens(10007, 150, 1), "q": H.random_tokens(10007, 67, 2), "s": H.random_tokens(10007, 40, 3)}
    want = {rid: plain.forward_logits(config_json, weights, toks).cpu() for rid, toks in requests.items()}
    for dtype in (torch.float32, torch.bfloat16):
        model = build_model(config).load(DictSource(weights), torch.device("cuda:0"), dtype)
        cache = CacheManager(model.cache_specs(), page_size=16, num_pages=40, max_requests=4, max_request_tokens=1024,
                             device=model.device, dtype=dtype)
        runner = ModelRunner(model, cache)
        # float32: the absolute bound of the other tests. bfloat16: these logits reach 6.5 where the tiny models'
        # reach 1.3, so the bound is relative: 2 % of the largest logit (rounding to 8 bits of mantissa at every
        # matrix-product input gives about 1 % here), and the mean error must stay below 2 % of the mean logit size.
        scale = max(float(w.abs().max()) for w in want.values())
        tol = 2e-4 if dtype == torch.float32 else 0.02 * scale
        if dtype == torch.bfloat16:
            got = H.replay(runner, H.cut_whole(requests))
            for rid, ref in want.items():
                assert float((got[rid] - ref).pow(2).mean().sqrt()) <= 0.02 * float(ref.pow(2).mean().sqrt()), rid
        H.assert_close(H.replay(runner, H.cut_whole(requests)), want, tol, f"real widths whole {dtype}")
        H.assert_close(H.replay(runner, H.cut_tail_one_by_one(requests, tail=32)), want, tol, f"real widths tail {dtype}")
        H.assert_close(H.replay(runner, H.cut_mixed(requests, (37, 2, 16, 64, 5), max_live=3)), want, tol, f"real widths mixed {dtype}")
        del runner, cache, model
        torch.cuda.empty_cache()


def write_trace(path, steps):
    with open(path, "w") as f:
        for i, (entries, end) in enumerate(steps):
            f.write(json.dumps({"step": i, "entries": [{"id": rid, "tokens": toks, "want": want} for rid, toks, want in entries],
                                "end": end}) + "\n")


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype_name):
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    tiny = plain.TINY_B
    folder, weights = H.make_case(tmp_path / "model", tiny, 1, dtype)
    requests = {f"q{i}": H.random_tokens(tiny["vocab_size"], n, 900 + i) for i, n in enumerate((33, 70, 12, 57, 41, 25))}
    steps = H.cut_mixed(requests, (7, 2, 16, 3, 5), max_live=4)
    steps.insert(3, ([], []))                                         # a step that brings nothing
    write_trace(tmp_path / "trace.jsonl", steps)
    out_dir = tmp_path / "out"
    with open(tmp_path / "trace.jsonl") as stdin:
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype_name,
                               "--out", str(out_dir), "--max-tokens", str(4 * 128)], stdin=stdin, capture_output=True,
                              text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    want = H.expected_logits(tiny, weights, requests)
    cursor = {rid: 0 for rid in requests}
    V = tiny["vocab_size"]
    for i, (entries, _end) in enumerate(steps):
        wanted = sum(len(w) for _, _, w in entries)
        path = out_dir / f"{i}.f32"
        if wanted == 0:
            assert not path.exists()
            continue
        data = torch.frombuffer(bytearray(path.read_bytes()), dtype=torch.float32).view(wanted, V)
        row = 0
        for rid, toks, w in entries:
            ref = want[rid][cursor[rid]:cursor[rid] + len(toks)][w]
            assert float((data[row:row + len(w)] - ref).abs().max()) <= H.TOL[dtype], (i, rid)
            row += len(w)
            cursor[rid] += len(toks)
    # the page ids the program wrote per step: a page that a finished request held is later held by another one
    held_by_finished = {}
    handed_on = 0
    for i, (entries, end) in enumerate(steps):
        if not entries:
            assert not (out_dir / f"{i}.pages.json").exists()
            continue
        pages = json.loads((out_dir / f"{i}.pages.json").read_text())["pages"]
        assert set(pages) == {rid for rid, _, _ in entries}
        for rid, tables in pages.items():
            assert len(tables[0]) == -(-cursor_after(steps, i, rid) // 16)
            for page in tables[0]:
                if page in held_by_finished and held_by_finished[page] != rid:
                    handed_on += 1
        for rid in end:
            for page in pages[rid][0]:
                held_by_finished[page] = rid
    assert handed_on > 0


def cursor_after(steps, upto, rid):
    return sum(len(toks) for entries, _ in steps[:upto + 1] for r, toks, _ in entries if r == rid)


def write_tokenizer(folder, vocab_size):
    """A word-level tokenizer.json with ``vocab_size`` entries and a tokenizer_config.json with a one-line chat template."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    words = ["<unk>", "<eos>"] + [f"w{i}" for i in range(vocab_size - 2)]
    tokenizer = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tokenizer.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tokenizer.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "unk_token": "<unk>",
                   "chat_template": "{% for m in messages %}w7 {{ m['content'] }} w8{% endfor %}"}, f)


def test_string_prompts_through_a_tokenizer(tmp_path):
    """The reference's public shape (src/llm_pipeline/inference/qwen3_engine.py:311-350, src/llm_pipeline/cli.py:24-41):
    a string in, a string out; a list of strings in, a list out; pieces of text from the stream; ``--prompt`` and
    ``--chat`` on the command line. The folder gets a tiny word-level tokenizer whose ids are the model's vocabulary."""
    tiny = plain.TINY_A
    folder, weights = H.make_case(tmp_path, tiny, 0, torch.float32, std=0.08)
    write_tokenizer(folder, tiny["vocab_size"])
    engine = engine_for(folder, torch.float32)
    assert engine.tokenizer is not None and engine.config.eos_token_id == 1
    ids = [5, 17, 3, 200, 9]
    text = " ".join(f"w{i - 2}" for i in ids)
    assert engine.tokenizer(text)["input_ids"] == ids
    want_ids = plain.greedy_generate(tiny, weights, ids, 6, eos_token_id=1)
    want = engine.tokenizer.decode(want_ids, skip_special_tokens=True)
    assert engine.generate(text, max_tokens=6, temperature=0.0) == want
    assert engine.generate([text, text], max_tokens=6, temperature=0.0) == [want, want]
    assert "".join(engine.stream_generate(text, max_tokens=6, temperature=0.0)) == want
    assert engine.engine.cache.num_live == 0
    base = [sys.executable, "-m", "llm_pipeline_b200.cli", "infer", "--model", folder, "--dtype", "fp32",
            "--max-new-tokens", "6", "--temperature", "0"]
    proc = subprocess.run(base + ["--prompt", text], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.strip() == want
    proc = subprocess.run(base + ["--prompt", text, "--chat"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    chat_ids = [9] + ids + [10]                                      # the template wraps the prompt in w7 ... w8
    assert proc.stdout.strip() == engine.tokenizer.decode(plain.greedy_generate(tiny, weights, chat_ids, 6, eos_token_id=1),
                                                          skip_special_tokens=True)


def test_a_stream_that_nobody_reads_to_the_end(tmp_path):
    """A caller that stops reading a stream leaves no request behind, and a generate call made while a stream is
    open waits for its own requests only."""
    tiny = plain.TINY_A
    folder, weights = H.make_case(tmp_path, tiny, 0, torch.float32, std=0.08)
    engine = engine_for(folder, torch.float32)
    prompt = H.random_tokens(256, 9, 77)
    stream = engine.stream_generate(prompt, max_tokens=5, temperature=0.0)
    first = next(stream)
    assert engine.engine.cache.num_live == 1
    other = H.random_tokens(256, 12, 78)
    got = engine.generate(other, max_tokens=12, temperature=0.0)      # the stream's request finishes during this call
    assert got == plain.greedy_generate(tiny, weights, other, 12)
    assert [first] + list(stream) == plain.greedy_generate(tiny, weights, prompt, 5)
    stream = engine.stream_generate(prompt, max_tokens=50, temperature=0.0)
    next(stream)
    stream.close()
    assert engine.engine.cache.num_live == 0 and not engine.engine.has_unfinished()


def test_cli_infer_with_token_ids(tmp_path):
    tiny = plain.TINY_A
    folder, weights = H.make_case(tmp_path, tiny, 0, torch.float32, std=0.08)
    prompt = [5, 17, 3, 200, 9]
    proc = subprocess.run([sys.executable, "-m", "llm_pipeline_b200.cli", "infer", "--model", folder, "--prompt-ids",
                           " ".join(map(str, prompt)), "--dtype", "fp32", "--max-new-tokens", "6", "--temperature", "0"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == plain.greedy_generate(tiny, weights, prompt, 6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_step_ahead_gives_what_reading_every_step_back_gives(tmp_path, dtype):
    """The engine plans and queues a step before it has read what the step before sampled (the ids go from the sampler
    to the next step on the device). The same tokens and finish reasons as with every step read back before the next is
    planned: with an end-of-sequence id that greedy generation meets (a request that stops was planned one step too
    far), with so few pages that requests are preempted while a token of theirs is in flight, with seeded sampling,
    and with a repetition penalty (which needs the tokens on the host: such steps are read back at once)."""
    tiny = plain.TINY_B
    folder, weights = H.make_case(tmp_path, tiny, 1, dtype, std=0.08)
    prompts = [H.random_tokens(tiny["vocab_size"], n, 640 + n) for n in (1, 33, 7, 52, 18, 26)]
    free = engine_for(folder, dtype, block_size=8, num_blocks=512).generate(prompts, max_tokens=30, temperature=0.0)
    flat = [t for out in free for t in out]
    eos = max(set(flat), key=flat.count)
    stops = preemptions = 0
    for blocks, kwargs in ((512, dict(temperature=0.0)), (14, dict(temperature=0.0)), (16, dict(temperature=0.8, top_k=0, top_p=1.0, seed=3)),
                           (512, dict(temperature=0.0, repetition_penalty=1.3))):
        outs = []
        for ahead in (False, True):
            # (in bfloat16 a preempted request's tokens are recomputed as a prompt, with other rounding than when they were
            # decoded, and the two ways of stepping preempt at different moments: few pages only in float32)
            engine = engine_for(folder, dtype, block_size=8, num_blocks=blocks if dtype == torch.float32 else 512, eos_token_id=eos,
                                max_batch_size=4, max_num_batched_tokens=32)
            engine.engine.lookahead = ahead
            results = engine.generate_ids(prompts, max_tokens=30, **kwargs)
            outs.append([(r.token_ids, r.finish_reason) for r in results])
            assert engine.engine.cache.num_live == 0 and not engine.engine.has_unfinished()
            engine.engine.cache.check()
            if ahead:
                preemptions += engine.engine.scheduler.num_preemptions
        assert outs[0] == outs[1], (blocks, kwargs)
        stops += sum(1 for _tokens, reason in outs[1] if reason == "stop")
        assert all(len(tokens) <= 30 and (reason != "stop" or tokens[-1] == eos) for tokens, reason in outs[1])
    assert stops >= 2 and (preemptions >= 1 or dtype != torch.float32)


@pytest.mark.parametrize("seed", [3, 8, 20])
def test_requests_that_arrive_and_are_aborted_while_the_engine_is_a_step_ahead(tmp_path, seed):
    """Requests added while others run (in their prompts, decoding, with a token in flight), some aborted on the way,
    few pages, seeded sampling and an end-of-sequence id: every request that is not aborted ends with the tokens and
    the reason it has when every step is read back before the next is planned; nothing is left in the cache."""
    import random
    from llm_pipeline_b200.sampling import SamplingConfig
    rng = random.Random(5000 + seed)
    tiny = plain.TINY_B
    folder, weights = H.make_case(tmp_path, tiny, seed, torch.float32, std=0.08)
    n = 10
    prompts = [H.random_tokens(tiny["vocab_size"], rng.randrange(1, 50), 300 + 13 * seed + i) for i in range(n)]
    limits = [rng.choice([1, 2, 5, 17, 30]) for _ in range(n)]
    arrive = sorted(rng.randrange(0, 25) for _ in range(n))                  # the step at which each request is added
    aborts = {i: arrive[i] + rng.randrange(1, 12) for i in range(n) if rng.random() < 0.3}
    free = engine_for(folder, torch.float32, block_size=8, num_blocks=512).generate(prompts, max_tokens=30, temperature=0.0)
    flat = [t for out in free for t in out]
    eos = max(set(flat), key=flat.count)
    outs = []
    for ahead in (False, True):
        engine = engine_for(folder, torch.float32, block_size=8, num_blocks=24, eos_token_id=eos, max_batch_size=4,
                            max_num_batched_tokens=24).engine
        engine.lookahead = ahead
        ids, step = {}, 0
        while len(ids) < n or engine.has_unfinished():
            for i in range(n):
                if i not in ids and arrive[i] <= step:
                    ids[i] = engine.add_request(prompts[i], max_tokens=limits[i], eos_token_ids=[eos],
                                                sampling=SamplingConfig(temperature=0.9, top_k=0, top_p=1.0, seed=7 + i))
            for i, at in aborts.items():
                if at == step and i in ids:
                    engine.abort(ids[i])
            if engine.has_unfinished():
                engine.step()
            step += 1
            assert step < 1000
        engine.drain()
        result = []
        for i in range(n):
            request = engine._requests[ids[i]]
            assert request.status == "finished" and request.in_flight == 0
            result.append((list(request.output) if request.finish_reason != "abort" else None, request.finish_reason))
        assert engine.cache.num_live == 0
        engine.cache.check()
        outs.append(result)
    for one, other in zip(*outs):
        assert one == other or "abort" in (one[1], other[1])
    assert any(reason == "abort" for _tokens, reason in outs[1]) and any(reason == "length" for _tokens, reason in outs[1])


def test_the_references_calls_around_its_batcher_and_caches(tmp_path):
    """qwen3_engine.py:614-712 under their names: requests that are added without waiting and asked for later, the
    counters of cache and scheduler, the switches, the model's sizes and parameter counts, the memory estimate."""
    tiny = plain.TINY_A
    folder, weights = H.make_case(tmp_path, tiny, 0, torch.float32, std=0.08)
    engine = engine_for(folder, torch.float32)
    engine.start_continuous_batching()
    prompts = [H.random_tokens(256, 9, 71), H.random_tokens(256, 21, 72)]
    ids = [engine.add_continuous_request(p, max_tokens=6, temperature=0.0) for p in prompts]
    assert len(set(ids)) == 2 and all(i.startswith("req_") for i in ids)
    results, polls = {}, 0
    while len(results) < 2:
        for i in ids:
            if i not in results:
                result = engine.get_continuous_result(i)
                if result is not None:
                    results[i] = result
        polls += 1
        assert polls < 200
    assert polls > 2                                            # the first questions found them unfinished
    for i, prompt in zip(ids, prompts):
        assert results[i]["generated_tokens"] == plain.greedy_generate(tiny, weights, prompt, 6)
        assert results[i]["tokens_generated"] == 6 and results[i]["prompt"] == prompt and results[i]["latency_ms"] > 0
        assert engine.get_continuous_result(i)["latency_ms"] == results[i]["latency_ms"]
    with pytest.raises(KeyError):
        engine.get_continuous_result("req_nobody")
    engine.stop_continuous_batching()
    assert engine.get_continuous_stats()["finished"] == 2 and engine.get_kv_cache_stats()["live_requests"] == 0
    switches = engine.get_optimization_stats()
    assert switches["paged_attention_enabled"] and switches["cuda_graphs_enabled"] and not switches["tensor_parallel_enabled"]
    info = engine.get_model_info()
    assert info["total_parameters"] == sum(t.numel() for t in weights.values()) and info["num_layers"] == tiny["num_hidden_layers"]
    memory = engine.estimate_memory_usage()
    assert memory["bytes_per_param"] == 4 and abs(memory["memory_mb"] - info["total_parameters"] * 4 / 2 ** 20) < 1e-9
    layers, kv_heads, head_dim = tiny["num_hidden_layers"], tiny["num_key_value_heads"], info["head_dim"]
    assert memory["kv_cache_bytes_per_token"] == layers * 2 * kv_heads * head_dim * 4
    engine.add_continuous_request(prompts[0], max_tokens=40)
    engine.engine.step()
    engine.clear_kv_cache()
    assert engine.get_kv_cache_stats()["live_requests"] == 0 and not engine.engine.has_unfinished()
