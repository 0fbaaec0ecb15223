"""The plain implementation against the outputs of the reference's own model code, which
tests/golden/make_golden.py recorded on the CPU (whole forward and its incremental cache path)."""

import json
import os

import pytest
import torch

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e"])
def test_plain_matches_recorded_reference_logits(name):
    with open(os.path.join(GOLDEN, f"{name}.json")) as f:
        gold = json.load(f)
    config = gold["config"]
    weights = plain.random_weights(config, gold["seed"])
    logits = plain.forward_logits(config, weights, gold["token_ids"])
    assert gold["plain_minus_reference_whole"] < 1e-5 and gold["plain_minus_reference_incremental"] < 1e-5
    for pos, row, arg in zip(gold["positions"], gold["logits"], gold["argmax"]):
        assert len(row) == config["vocab_size"]
        assert torch.allclose(logits[pos], torch.tensor(row), atol=2e-6, rtol=0)
        assert int(logits[pos].argmax()) == arg
    assert abs(float(logits.abs().max()) - gold["max_abs_logit"]) < 1e-5


def test_logits_at_a_position_do_not_depend_on_later_tokens():
    w = plain.random_weights(plain.TINY_A, 0)
    ids = list(range(3, 40))
    full = plain.forward_logits(plain.TINY_A, w, ids)
    part = plain.forward_logits(plain.TINY_A, w, ids[:17])
    assert torch.allclose(full[:17], part, atol=1e-6)


def test_float64_agrees_with_float32():
    w = plain.random_weights(plain.TINY_B, 1)
    ids = list(range(1, 30))
    a = plain.forward_logits(plain.TINY_B, w, ids, dtype=torch.float32)
    b = plain.forward_logits(plain.TINY_B, w, ids, dtype=torch.float64)
    assert float((a - b.float()).abs().max()) < 1e-5


def test_sampler_filters():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0, 0.0])
    assert plain.apply_top_k(logits, 2).isfinite().tolist() == [True, False, False, False, True, False]
    kept = plain.apply_top_p(logits, 0.8).isfinite().tolist()
    assert kept == [True, False, False, False, True, False]      # 0.61 then 0.84 crosses 0.8: two kept
    assert plain.apply_min_p(logits, 0.3).isfinite().tolist() == [True, False, False, False, True, False]
    pen = plain.apply_repetition_penalty(logits, [0, 3, 3], 2.0)
    assert pen.tolist() == [1.0, 1.0, 0.5, -2.0, 3.0, 0.0]
    probs = plain.filtered_probs(logits, temperature=0.7, top_k=3, top_p=0.95)
    assert abs(float(probs.sum()) - 1) < 1e-6 and int((probs > 0).sum()) <= 3
    assert plain.inverse_cdf_pick(torch.tensor([0.2, 0.3, 0.5]), 0.1) == 0
    assert plain.inverse_cdf_pick(torch.tensor([0.2, 0.3, 0.5]), 0.49) == 1
    assert plain.inverse_cdf_pick(torch.tensor([0.2, 0.3, 0.5]), 0.9999) == 2
