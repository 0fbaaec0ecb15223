"""Weights: names and shapes are checked as a whole; random model folders round-trip."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_qwen3 as plain
from llm_pipeline_b200.config import resolve_config
from llm_pipeline_b200.models import build_model
from llm_pipeline_b200.weights import (DictSource, SafetensorsSource, WeightError, check_names_and_shapes,
                                       stored_dtype_policy, write_random_model)


@pytest.mark.parametrize("tiny", [plain.TINY_A, plain.TINY_B, plain.TINY_C])
def test_expected_names_are_the_reference_names(tiny):
    expected = build_model(resolve_config(tiny)).expected_params()
    names = {n for n, s in expected.items() if not s.optional}
    assert names == set(plain.tensor_shapes(tiny))
    for name, shape in plain.tensor_shapes(tiny).items():
        assert tuple(expected[name].shape) == tuple(shape)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    expected = build_model(resolve_config(plain.TINY_B)).expected_params()
    w = plain.random_weights(plain.TINY_B, 1)
    del w["model.norm.weight"], w["model.layers.2.self_attn.k_norm.weight"]
    w["model.layers.0.mlp.extra.weight"] = torch.zeros(2)
    w["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(5, 7)
    w["model.rotary_emb.inv_freq"] = torch.zeros(16)            # a known non-parameter: ignored
    with pytest.raises(WeightError) as e:
        check_names_and_shapes(expected, DictSource(w))
    err = e.value
    assert sorted(err.missing) == ["model.layers.2.self_attn.k_norm.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert err.wrong_shape == [("model.layers.1.self_attn.q_proj.weight", (5, 7), (192, 96))]
    text = str(err)
    for fragment in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[5, 7], expected [192, 96]"):
        assert fragment in text


def test_tied_head_is_optional_and_untied_head_is_required():
    tied = build_model(resolve_config(plain.TINY_A)).expected_params()
    w = plain.random_weights(plain.TINY_A, 0)
    check_names_and_shapes(tied, DictSource(w))
    check_names_and_shapes(tied, DictSource({**w, "lm_head.weight": w["model.embed_tokens.weight"]}))
    untied = build_model(resolve_config(plain.TINY_B)).expected_params()
    w = plain.random_weights(plain.TINY_B, 1)
    del w["lm_head.weight"]
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_names_and_shapes(untied, DictSource(w))


def test_a_copy_of_a_tied_head_must_repeat_the_embedding():
    # The reference's tied head is the embedding's own tensor (models/qwen3/custom_builder.py:389-391): a checkpoint
    # that holds other values under lm_head.weight contradicts its configuration, and loading says so.
    from llm_pipeline_b200.weights import TiedWeightError
    w = plain.random_weights(plain.TINY_A, 0)
    model = build_model(resolve_config(plain.TINY_A))
    model.load(DictSource({**w, "lm_head.weight": w["model.embed_tokens.weight"].clone()}), torch.device("cpu"), torch.float32)
    assert model.head.weight is model.embedding.weight
    with pytest.raises(TiedWeightError, match="lm_head.weight differs from model.embed_tokens.weight"):
        build_model(resolve_config(plain.TINY_A)).load(
            DictSource({**w, "lm_head.weight": w["model.embed_tokens.weight"] + 1.0}), torch.device("cpu"), torch.float32)


def test_random_model_folder_round_trips(tmp_path):
    folder = write_random_model(plain.TINY_C, seed=7, out_dir=str(tmp_path / "m"), dtype=torch.bfloat16)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    with open(os.path.join(folder, "config.json")) as f:
        assert json.load(f)["head_dim"] == 48
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    assert set(tensors) == set(plain.tensor_shapes(plain.TINY_C))
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    norm = tensors["model.layers.0.input_layernorm.weight"].float()
    assert 0.7 < float(norm.mean()) < 1.3 and float(tensors["model.embed_tokens.weight"].float().std()) < 0.03
    again = load_file(os.path.join(write_random_model(plain.TINY_C, 7, str(tmp_path / "n")), "model.safetensors"))
    other = load_file(os.path.join(write_random_model(plain.TINY_C, 8, str(tmp_path / "o")), "model.safetensors"))
    assert all(torch.equal(tensors[k], again[k]) for k in tensors)
    assert not torch.equal(tensors["lm_head.weight"], other["lm_head.weight"])
    src = SafetensorsSource(folder)
    check_names_and_shapes(build_model(resolve_config(plain.TINY_C)).expected_params(), src)
    src.close()


def test_sharded_folders_and_duplicates(tmp_path):
    w = plain.random_weights(plain.TINY_A, 0)
    names = sorted(w)
    save_file({k: w[k] for k in names[:10]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: w[k] for k in names[10:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    src = SafetensorsSource(str(tmp_path))
    check_names_and_shapes(build_model(resolve_config(plain.TINY_A)).expected_params(), src)
    assert torch.equal(src.get(names[12]), w[names[12]])
    src.close()
    save_file({names[0]: w[names[0]]}, str(tmp_path / "zz.safetensors"))
    with pytest.raises(WeightError, match="stored twice"):
        SafetensorsSource(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        SafetensorsSource(str(tmp_path / "empty"))


def test_storage_types():
    bf, f32 = torch.bfloat16, torch.float32
    assert stored_dtype_policy("matrix", bf, bf) == bf
    assert stored_dtype_policy("matrix", f32, bf) == bf          # a matrix product operand takes the compute type
    assert stored_dtype_policy("vector", f32, bf) == f32         # stored in 32-bit: stays so
    assert stored_dtype_policy("vector", bf, bf) == bf
    assert stored_dtype_policy("matrix", bf, f32) == f32 and stored_dtype_policy("vector", bf, f32) == f32
    assert stored_dtype_policy("table", torch.int64, bf) == torch.int32
