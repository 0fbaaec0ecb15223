"""Seeded random configurations of the architecture, each replayed as a mixed trace with page reuse, in
float32 and in bfloat16, against the plain implementation. Half of them have head size 128, the size
that the tcgen05 prefill attention and the TMA decode stream serve in bfloat16, with every group size
from 1 to 8 and some above."""

import random

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    head_dim = 128 if seed % 2 == 0 else rng.choice([16, 32, 48, 64, 80, 96, 112])
    group = (seed // 2) % 8 + 1 if seed % 2 == 0 else rng.choice([1, 2, 3, 5, 12])
    if seed == 8:
        group = 16                                           # above the decode stream's 8 heads per group
    kv_heads = rng.choice([1, 2, 3])
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
        "num_hidden_layers": rng.choice([1, 2, 3]),
        "hidden_size": rng.choice([72, 96, 136, 200, 264]),          # multiples of 8, no powers of two
        "num_attention_heads": kv_heads * group, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": rng.choice([88, 152, 232, 328]),
        "vocab_size": rng.choice([257, 300, 512, 777]),
        "rope_theta": rng.choice([10000.0, 500000.0, 1000000.0]),
        "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6]),
        "tie_word_embeddings": rng.random() < 0.5, "attention_bias": rng.random() < 0.3,
        "max_position_embeddings": 2048, "hidden_act": "silu",
    }


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(12))
def test_random_configuration_mixed_trace(tmp_path, seed, dtype):
    config = random_config(seed)
    rng = random.Random(1000 + seed)
    page = rng.choice([8, 16, 32])
    folder, weights = H.make_case(tmp_path, config, seed, dtype)
    lengths = [rng.choice([1, 2, 3, 17, 40, 130, 200, 290]) for _ in range(6)] + [rng.randrange(120, 300)]
    requests = {f"r{i}": H.random_tokens(config["vocab_size"], n + 7, 2000 + 10 * seed + i) for i, n in enumerate(lengths)}
    want = H.expected_logits(config, weights, requests)
    longest = max(len(t) for t in requests.values())
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=4 * (-(-longest // page)))
    sizes = [rng.choice([2, 3, 5, 16, 31, 64, 129]) for _ in range(5)]
    got = H.replay(runner, H.cut_mixed(requests, sizes, max_live=4))
    H.assert_close(got, want, H.TOL[dtype], f"random configuration {seed} ({config})")
    assert runner.cache.num_live == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_configuration_with_widths_in_multiples_of_64(tmp_path, seed):
    """Widths that the streaming products of a decode step take, so that steps of up to 8 tokens fold their norms into
    the products around them (and steps of more tokens do not): token by token, in small portions and mixed."""
    dtype = torch.bfloat16
    rng = random.Random(500 + seed)
    config = dict(random_config(seed), hidden_size=rng.choice([64, 128, 192, 320]), intermediate_size=rng.choice([64, 192, 448]),
                  head_dim=rng.choice([64, 128]))
    page = rng.choice([8, 16, 32])
    folder, weights = H.make_case(tmp_path, config, seed, dtype)
    lengths = [rng.choice([1, 2, 9, 17, 40, 130]) for _ in range(5)] + [rng.randrange(120, 260)]
    requests = {f"r{i}": H.random_tokens(config["vocab_size"], n + 7, 3000 + 10 * seed + i) for i, n in enumerate(lengths)}
    want = H.expected_logits(config, weights, requests)
    longest = max(len(t) for t in requests.values())
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=4 * (-(-longest // page)))
    from llm_pipeline_b200.ops import kernels
    folded, launch, launch_chain = [], kernels.gemm_stream_fused, kernels.gemm_stream_chain

    def counting(*args, **kwargs):
        folded.append(1)
        return launch(*args, **kwargs)

    def counting_chain(*args, **kwargs):
        folded.append(len(args[0]))
        return launch_chain(*args, **kwargs)

    kernels.gemm_stream_fused, kernels.gemm_stream_chain = counting, counting_chain
    try:
        H.assert_close(H.replay(runner, H.cut_portions(requests, (1,))), want, H.TOL[dtype], f"token by token ({config})")
        H.assert_close(H.replay(runner, H.cut_portions(requests, (3, 8, 2, 9))), want, H.TOL[dtype], f"portions ({config})")
        H.assert_close(H.replay(runner, H.cut_mixed(requests, (2, 3, 5, 16), max_live=4)), want, H.TOL[dtype], f"mixed ({config})")
    finally:
        kernels.gemm_stream_fused, kernels.gemm_stream_chain = launch, launch_chain
    # a product with a bias is not handed to the norm, and the last layer's goes to the final norm as a tensor
    assert folded or (config["attention_bias"] and config["num_hidden_layers"] == 1)
    assert runner.cache.num_live == 0
