"""The engine against the plain implementation under every way of cutting the work, in float32
and in bfloat16, at tiny configurations that differ in every size and option."""

import pytest
import torch

import helpers as H
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

CASES = [
    pytest.param(plain.TINY_A, 0, 16, (5, 17, 33), id="tiny_a"),
    pytest.param(plain.TINY_B, 1, 8, (1, 9, 24, 40), id="tiny_b"),
    pytest.param(plain.TINY_C, 2, 16, (3, 50, 21), id="tiny_c"),
    pytest.param(plain.TINY_D, 3, 16, (133, 9, 262), id="tiny_d"),       # crosses the 128-key tiles of attention
    pytest.param(plain.TINY_E, 4, 8, (7, 30, 61), id="tiny_e"),          # decode steps fold the norms into the products
]
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def _requests(config, lengths, extra=8):
    return {f"r{i}": H.random_tokens(config["vocab_size"], n + extra, 1000 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("config,seed,page,lengths", CASES)
def test_cuts_match_plain(tmp_path, config, seed, page, lengths, dtype):
    folder, weights = H.make_case(tmp_path, config, seed, dtype)
    requests = _requests(config, lengths)
    want = H.expected_logits(config, weights, requests)
    tol = H.TOL[dtype]
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=64)
    H.assert_close(H.replay(runner, H.cut_whole(requests)), want, tol, "whole")
    H.assert_close(H.replay(runner, H.cut_tail_one_by_one(requests, tail=32)), want, tol, "tail one by one")
    H.assert_close(H.replay(runner, H.cut_portions(requests, (7, 2, 16, 3, 5))), want, tol, "portions")
    H.assert_close(H.replay(runner, H.cut_portions(requests, (1,))), want, tol, "token by token")
    assert runner.cache.num_live == 0
    assert runner.use_graphs and runner.graph_replays > 0       # single-token steps ran as replayed CUDA graphs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("config,seed,page,lengths", CASES)
def test_mixed_batches_with_page_reuse(tmp_path, config, seed, page, lengths, dtype):
    folder, weights = H.make_case(tmp_path, config, seed, dtype)
    lengths = tuple(lengths) + (29, 12, 44, 7)
    requests = _requests(config, lengths)
    want = H.expected_logits(config, weights, requests)
    # pages for four live requests of the longest length, and no more: later requests reuse pages
    longest = max(len(t) for t in requests.values())
    num_pages = 4 * (-(-longest // page))
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=num_pages)
    got = H.replay(runner, H.cut_mixed(requests, (7, 2, 16, 3, 5), max_live=4))
    H.assert_close(got, want, H.TOL[dtype], "mixed")
    assert runner.cache.pages_reused > 0
    assert runner.cache.num_live == 0


def test_decode_of_uneven_batch_shares_the_long_request(tmp_path, monkeypatch):
    """One request far longer than the others: the decode steps (eager, then as a replayed graph) take the attention
    kernel that deals key ranges out over all SMs (forced here: at this tiny size the other one would be chosen);
    logits as from the plain implementation."""
    from llm_pipeline_b200.ops import kernels
    monkeypatch.setattr(kernels, "_DECODE_LIST", "1")
    dtype = torch.bfloat16
    folder, weights = H.make_case(tmp_path, plain.TINY_D, 5, dtype)
    requests = _requests(plain.TINY_D, (1700, 20, 60), extra=10)
    want = H.expected_logits(plain.TINY_D, weights, requests)
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=160)
    tail = 10
    steps = [([(rid, toks[:-tail], list(range(len(toks) - tail)))], []) for rid, toks in requests.items()]
    for i in range(tail):
        at = {rid: len(toks) - tail + i for rid, toks in requests.items()}
        steps.append(([(rid, [toks[at[rid]]], [0]) for rid, toks in requests.items()], list(requests) if i == tail - 1 else []))
    H.assert_close(H.replay(runner, steps), want, H.TOL[dtype], "uneven decode")
    assert runner.graph_replays > 0 and runner.cache.num_live == 0
    kernels.check_error_flag()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("config,seed,page,lengths", CASES)
def test_mixed_batches_with_decoded_tokens_through_the_decode_kernel(tmp_path, monkeypatch, config, seed, page, lengths, dtype):
    """In a step that mixes decoded tokens with portions of prompts, the single-token requests at its front go through
    the decode kernel once one of them has a long context; here always, with the decoding requests put first as the scheduler
    does."""
    from llm_pipeline_b200.parts.attention import AttentionPolicy
    monkeypatch.setattr(AttentionPolicy, "SPLIT_DECODE_MIN_CONTEXT", 0)
    folder, weights = H.make_case(tmp_path, config, seed, dtype)
    requests = _requests(config, tuple(lengths) + (29, 12, 44, 7))
    want = H.expected_logits(config, weights, requests)
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=4 * (-(-max(len(t) for t in requests.values()) // page)))
    steps = [(sorted(entries, key=lambda e: len(e[1]) != 1), end)
             for entries, end in H.cut_mixed(requests, (7, 2, 16, 3, 5), max_live=4, decode_tail=12)]
    assert any(len(entries[0][1]) == 1 and len(entries[-1][1]) > 1 for entries, _ in steps)
    H.assert_close(H.replay(runner, steps), want, H.TOL[dtype], "mixed, decode kernel for single tokens")
    assert runner.cache.num_live == 0


def test_prompt_portions_whose_tiles_share_their_keys(tmp_path, monkeypatch):
    """Long contexts make the work list of the tcgen05 attention kernel cut a tile's keys into items; here from the
    second key tile on, so that the tiny model's portions take that path: portions of changing size and mixed steps."""
    from llm_pipeline_b200.ops import kernels
    from llm_pipeline_b200.parts.attention import AttentionPolicy
    monkeypatch.setattr(AttentionPolicy, "SPLIT_KEYS_MIN_TILES", 1)
    shared, launch = [], kernels.paged_attention

    def counting(*args, **kwargs):
        shared.append(args[18] if len(args) > 18 else kwargs.get("places", 0))
        return launch(*args, **kwargs)

    monkeypatch.setattr(kernels, "paged_attention", counting)
    dtype = torch.bfloat16
    folder, weights = H.make_case(tmp_path, plain.TINY_D, 7, dtype)
    requests = _requests(plain.TINY_D, (533, 9, 262, 700))
    want = H.expected_logits(plain.TINY_D, weights, requests)
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=128)
    H.assert_close(H.replay(runner, H.cut_whole(requests)), want, H.TOL[dtype], "whole")
    H.assert_close(H.replay(runner, H.cut_portions(requests, (70, 2, 160, 33, 5))), want, H.TOL[dtype], "portions")
    H.assert_close(H.replay(runner, H.cut_mixed(requests, (70, 2, 160, 33, 5), max_live=4)), want, H.TOL[dtype], "mixed")
    assert runner.cache.num_live == 0 and max(shared) > 0
    kernels.check_error_flag()


def test_which_decode_kernel_a_step_takes():
    """Blocks of its own for every request while contexts are even; key ranges dealt out evenly when one request would
    keep its blocks reading long after the others, or when requests are many (Qwen3-8B heads on the GPU's SMs)."""
    from llm_pipeline_b200.ops import kernels

    def takes_list(contexts, kv_heads=8):
        return kernels.decode_prefers_list(max(contexts), sum(contexts), len(contexts), kv_heads)

    assert not takes_list([2048]) and not takes_list([2048] * 8) and not takes_list([16384] * 8) and not takes_list([2048] * 32)
    assert takes_list([131072]) and takes_list([32768, 600]) and takes_list([16384] + [512] * 7) and takes_list([2048] * 64)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_request_name_that_comes_back_gets_its_own_block_table(tmp_path, dtype):
    """A request ends and a new one arrives under the same name, on other pages: replayed decode graphs keep the
    rows of their last step's requests and rewrite only what moved, so they must tell the two apart."""
    config = plain.TINY_A
    folder, weights = H.make_case(tmp_path, config, 11, dtype)
    first = {"a": H.random_tokens(config["vocab_size"], 40, 1)}
    second = {"a": H.random_tokens(config["vocab_size"], 40, 2), "b": H.random_tokens(config["vocab_size"], 30, 3)}
    runner = H.make_runner(folder, dtype, page_size=8, num_pages=32)
    H.assert_close(H.replay(runner, H.cut_portions(first, (1,))), H.expected_logits(config, weights, first), H.TOL[dtype], "first")
    steps = [([("b", second["b"][:29], [28])], [])]                   # b takes the pages that a had
    # a again: most of it as one portion, so that its first single-token step finds the graph of the first a's last
    # steps, with a block table as long as the one remembered there
    steps.append(([("a", second["a"][:33], [32])], []))
    for i in range(33, 40):
        steps.append(([("a", [second["a"][i]], [0])], ["a"] if i == 39 else []))
    steps.append(([("b", second["b"][29:], [0])], ["b"]))
    want = H.expected_logits(config, weights, second)
    got = H.replay(runner, steps)
    assert torch.allclose(got["a"], want["a"][32:], atol=H.TOL[dtype]), float((got["a"] - want["a"][32:]).abs().max())
    assert torch.allclose(got["b"], want["b"][28:], atol=H.TOL[dtype])
    assert runner.graph_replays > 0 and runner.cache.num_live == 0


NEEDLE_CONFIG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 256,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 512, "vocab_size": 384,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 2048, "hidden_act": "silu",
}


def test_a_planted_far_key_through_the_decode_graph_in_bfloat16(tmp_path):
    """Random weights spread a softmax over hundreds of keys, and a far key that a kernel drops changes the logits by
    less than bfloat16 rounding does. Here the embedding of one token is made so that, as the first token of a long
    prompt, its key in the first layer is exactly what the decoded token's query looks for at one position (cosine 1
    where random keys reach 0.3): one head's attention sits on the key at position 0, in the first page, hundreds of
    keys away. The step that must find it runs head size 128 in bfloat16 as a replayed graph with the norms folded
    into the streaming products, beside two other requests; without the key the oracle's logits differ by many times
    the tolerance, so a kernel that lost it would fail."""
    cfg = NEEDLE_CONFIG
    dtype = torch.bfloat16
    d, H_, nkv = cfg["head_dim"], cfg["hidden_size"], cfg["num_key_value_heads"]
    weights = plain.random_weights(cfg, 21, std=0.05)
    needle, query_token, far = 7, 11, 600                       # token ids; the query's position
    # the query of head 0 of the first layer for `query_token` at position `far`
    x = plain.rms_norm(weights["model.embed_tokens.weight"][query_token], weights["model.layers.0.input_layernorm.weight"], 1e-6)
    q = (weights["model.layers.0.self_attn.q_proj.weight"] @ x)[:d]
    q = plain.rms_norm(q, weights["model.layers.0.self_attn.q_norm.weight"], 1e-6)
    cos, sin = plain.rope_cos_sin(torch.tensor([far]), d, cfg["rope_theta"])
    target = plain.apply_rope(q[None, None, :], cos, sin)[0, 0]            # the key at position 0 is not rotated
    # an embedding whose key (head 0 of the key/value heads) is parallel to the target: Wk (ln1 * e / rms) ~ target / k_norm
    wk = weights["model.layers.0.self_attn.k_proj.weight"][:d]
    wanted = target / weights["model.layers.0.self_attn.k_norm.weight"]
    e = torch.linalg.pinv(wk) @ wanted / weights["model.layers.0.input_layernorm.weight"]
    weights["model.embed_tokens.weight"][needle] = e * (0.05 * H_ ** 0.5 / e.norm())
    weights = {k: v.to(dtype).float() for k, v in weights.items()}
    folder = H.write_model_dir(str(tmp_path), cfg, weights, dtype)

    filler = [t for t in H.random_tokens(cfg["vocab_size"], far + 40, 77) if t not in (needle, query_token)][:far - 1]
    with_key = [needle] + filler + [query_token] * 4             # the query token lands on positions far .. far + 3
    without = [filler[5]] + filler + [query_token] * 4
    want = plain.forward_logits(cfg, weights, with_key, dtype=torch.float64).float()[far:]
    blind = plain.forward_logits(cfg, weights, without, dtype=torch.float64).float()[far:]
    tol = H.TOL[dtype] * max(1.0, float(want.abs().max()))          # the bound of the tiny models (logits up to 1), scaled to these logits (2)
    assert float((want[0] - blind[0]).abs().max()) > 8 * tol        # the key matters far more than rounding does

    from llm_pipeline_b200.engine import StepEntry
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=128, max_request_tokens=1024)
    others = {"u": H.random_tokens(cfg["vocab_size"], 150, 5), "v": H.random_tokens(cfg["vocab_size"], 33, 6)}
    for rid, toks in others.items():
        runner.step([StepEntry(rid, toks[:-8], [])])
    for at in range(0, far, 97):                                   # the prompt in portions that cross the 128-key tiles
        runner.step([StepEntry("n", with_key[at:min(at + 97, far)], [])])
    rows = []
    for s in range(4):                                             # eager, captured, replayed, replayed
        entries = [StepEntry("u", [others["u"][-8 + s]], []), StepEntry("n", [with_key[far + s]], [0]), StepEntry("v", [others["v"][-8 + s]], [])]
        rows.append(runner.step(entries)[0].float().cpu().clone())
    got = torch.stack(rows)
    assert runner.graph_replays >= 2
    assert float((got - want).abs().max()) <= tol, float((got - want).abs().max())
    assert float((got[0] - blind[0]).abs().max()) > 6 * tol
    from llm_pipeline_b200.ops import kernels
    kernels.check_error_flag()


def test_kernel_times_and_nvtx_ranges_of_steps(tmp_path, monkeypatch):
    """CUDA events around every launch (``ops.timing.KernelTimes``): as a block around one step, and for every step of
    a runner when the switch is on (graphs are then off); with NVTX ranges pushed around step, layers and head. The
    logits are what they are without any of it."""
    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.ops import timing
    tiny = plain.TINY_D
    folder, weights = H.make_case(tmp_path, tiny, 3, torch.bfloat16)
    layers = tiny["num_hidden_layers"]
    runner = H.make_runner(folder, torch.bfloat16, page_size=16, num_pages=16)
    tokens = H.random_tokens(tiny["vocab_size"], 40, 9)
    plain_logits = runner.step([StepEntry("a", tokens, [39])]).float().cpu()
    runner.release("a")
    monkeypatch.setattr(timing, "NVTX", True)
    with timing.KernelTimes() as times:
        timed_logits = runner.step([StepEntry("a", tokens, [39])]).float().cpu()
    assert torch.equal(plain_logits, timed_logits)
    table = times.table()
    assert table["qkv_post"]["launches"] == layers and table["paged_attention"]["launches"] == layers
    assert table["embedding"]["launches"] == 1 and all(row["us"] > 0 for row in table.values())
    products = sum(row["launches"] for name, row in table.items() if row["flops"] > 0)
    assert products == 4 * layers + 1                       # q/k/v, output, gate/up, down per layer; the head
    assert list(table) == sorted(table, key=lambda name: -table[name]["us"])
    runner.release("a")
    # the switch: every step of a new runner is timed, none is captured
    monkeypatch.setattr(timing, "TIME_KERNELS", True)
    timed = H.make_runner(folder, torch.bfloat16, page_size=16, num_pages=16)
    assert timed.kernel_times is not None and not timed.use_graphs
    timed.step([StepEntry("b", tokens, [])])
    for i in range(4):
        timed.step([StepEntry("b", [tokens[i]], [0])])
    totals = timed.kernel_times.table()
    assert totals["decode_attention"]["launches"] == 4 * layers and totals["paged_attention"]["launches"] == layers
    assert timed.graph_replays == 0


@pytest.mark.parametrize("config,seed", [(plain.TINY_A, 0), (plain.TINY_D, 3)], ids=["a", "d"])
def test_prompt_portions_whose_products_add_themselves_into_the_residual(tmp_path, monkeypatch, config, seed):
    """Many rows of a large matrix leave the sum of residual and product to the library's product (float32 C operand).
    With the limits lowered so that the tiny models take that way: whole prompts, portions on both sides of the limit
    and mixed batches give the plain implementation's logits, and the way was taken."""
    import importlib
    linear = importlib.import_module("llm_pipeline_b200.ops.linear")
    from llm_pipeline_b200.ops import kernels
    monkeypatch.setattr(linear, "ACCUMULATE_MIN_ROWS", 16)
    monkeypatch.setattr(linear, "ACCUMULATE_MIN_WEIGHTS", 0)
    calls = []
    real = kernels.library_add_product
    monkeypatch.setattr(kernels, "library_add_product", lambda r, x, w: calls.append(x.shape[0]) or real(r, x, w))
    folder, weights = H.make_case(tmp_path, config, seed, torch.bfloat16)
    runner = H.make_runner(folder, torch.bfloat16, page_size=16, num_pages=24)
    requests = {f"r{i}": H.random_tokens(config["vocab_size"], n, 900 + i) for i, n in enumerate((70, 17, 45, 33))}
    want = H.expected_logits(config, weights, requests)
    tol = H.TOL[torch.bfloat16]
    H.assert_close(H.replay(runner, H.cut_whole(requests)), want, tol, "accumulate whole")
    assert calls and min(calls) >= 16
    whole = len(calls)
    H.assert_close(H.replay(runner, H.cut_portions(requests, (20, 5, 16, 31))), want, tol, "accumulate portions")
    H.assert_close(H.replay(runner, H.cut_mixed(requests, (18, 3, 40, 16), max_live=3)), want, tol, "accumulate mixed")
    assert len(calls) > whole and min(calls) >= 16
    # where the library's call cannot be had (it answers False), the product is taken and added as everywhere else
    monkeypatch.setattr(kernels, "library_add_product", lambda r, x, w: False)
    H.assert_close(H.replay(runner, H.cut_whole(requests)), want, tol, "accumulate refused")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_context_of_several_thousand_tokens_in_portions_and_decoded(tmp_path, dtype):
    """A request of 6,300 tokens at head size 128 beside a short one: the prompt in portions of 2,048, 1,500, 37 and 2
    tokens (a few new tokens over thousands of cached keys: in bfloat16 the tiles of such a portion share their keys),
    then tokens decoded one by one beside the other request's (the longer request is read by many SMs), against the
    plain implementation in float64 on the same device, at the last place of every portion and at every decoded one."""
    from llm_pipeline_b200.engine import StepEntry
    config = dict(plain.TINY_D, max_position_embeddings=8192)
    folder, weights = H.make_case(tmp_path, config, 5, dtype)
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=420, max_request_tokens=6400)
    long_ids, short_ids = H.random_tokens(config["vocab_size"], 6300, 71), H.random_tokens(config["vocab_size"], 150, 72)
    cuts = [2048, 2048, 1500, 600, 37, 2, 57]                       # 6,292 tokens of prompt, then 8 decoded
    assert sum(cuts) == 6292
    got, rows, done = [], [], 0
    for i, n in enumerate(cuts):
        entries = [StepEntry("long", long_ids[done:done + n], [n - 1])]
        if i == 3:
            entries.append(StepEntry("short", short_ids[:142], []))                  # joins in the middle of the long prompt
        got.append(runner.step(entries).float().cpu())
        done += n
        rows.append(done - 1)
    for i in range(8):
        logits = runner.step([StepEntry("long", [long_ids[6292 + i]], [0]), StepEntry("short", [short_ids[142 + i]], [0])])
        got.append(logits[:1].float().cpu())
        rows.append(6292 + i)
        short_row = logits[1:].float().cpu()
    device_weights = {k: v.cuda() for k, v in weights.items()}
    want = plain.forward_logits(config, device_weights, long_ids, dtype=torch.float64, rows=rows).float().cpu()
    want_short = plain.forward_logits(config, device_weights, short_ids, dtype=torch.float64, rows=[149]).float().cpu()
    tol = H.TOL[dtype] * max(1.0, float(want.abs().max()))
    worst = float((torch.cat(got) - want).abs().max())
    assert worst <= tol, (worst, tol)
    assert float((short_row - want_short).abs().max()) <= tol
    assert runner.graph_replays >= 5
    runner.release("long")
    runner.release("short")
    runner.cache.check()
    assert runner.cache.num_live == 0
