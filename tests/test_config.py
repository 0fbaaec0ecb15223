"""Typed configuration and the architecture registry."""

import json
import warnings

import pytest

import plain_qwen3 as plain
from llm_pipeline_b200.config import (ModelConfig, Qwen3Config, load_config, register_architecture, resolve_config,
                                      supported_architectures)


def test_qwen3_config_reads_every_size_from_json():
    for tiny in (plain.TINY_A, plain.TINY_B, plain.TINY_C):
        cfg = resolve_config(tiny)
        assert isinstance(cfg, Qwen3Config)
        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                    "head_dim", "intermediate_size", "rms_norm_eps", "rope_theta", "tie_word_embeddings",
                    "attention_bias", "max_position_embeddings"):
            assert getattr(cfg, key) == tiny[key], key
        spec = cfg.model_spec()
        assert len(spec.layers) == tiny["num_hidden_layers"] == len(spec.schedule)
        attn = spec.layers[0].mixer.args
        assert attn["num_heads"] == tiny["num_attention_heads"] and attn["head_dim"] == tiny["head_dim"]
        assert attn["scale"] == tiny["head_dim"] ** -0.5 and attn["window"] is None
        assert spec.head.args["tied_to"] == ("model.embed_tokens" if tiny["tie_word_embeddings"] else None)


def test_defaults_follow_the_reference_model_code():
    d = {k: v for k, v in plain.TINY_A.items() if k not in ("head_dim", "rope_theta", "rms_norm_eps", "attention_bias",
                                                            "tie_word_embeddings")}
    cfg = resolve_config(d)
    assert cfg.head_dim == d["hidden_size"] // d["num_attention_heads"]
    assert cfg.rope_theta == 1000000.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.attention_bias is False and cfg.tie_word_embeddings is False


def test_aliases_and_nested_rope():
    d = dict(plain.TINY_B)
    d["num_layers"] = d.pop("num_hidden_layers")
    d["norm_epsilon"] = d.pop("rms_norm_eps")
    d["rope_parameters"] = {"rope_theta": d.pop("rope_theta"), "rope_type": "default"}
    cfg = resolve_config(d)
    assert cfg.num_hidden_layers == 3 and cfg.num_layers == 3
    assert cfg.rms_norm_eps == 1e-5 and cfg.norm_epsilon == 1e-5 and cfg.rope_theta == 1000000.0


def test_missing_and_invalid_keys_are_named():
    d = dict(plain.TINY_A)
    del d["intermediate_size"], d["vocab_size"]
    with pytest.raises(ValueError, match="intermediate_size") as e:
        resolve_config(d)
    assert "vocab_size" in str(e.value)
    with pytest.raises(ValueError, match="not a multiple"):
        resolve_config({**plain.TINY_A, "num_key_value_heads": 3})
    with pytest.raises(ValueError, match="even"):
        resolve_config({**plain.TINY_A, "head_dim": 15})


def test_ignored_keys_warn():
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        cfg = resolve_config({**plain.TINY_A, "use_sliding_window": True, "sliding_window": 8,
                              "rope_scaling": {"rope_type": "yarn", "factor": 4.0}, "hidden_act": "gelu"})
    assert len(w) == 3
    assert all(layer.mixer.args["window"] is None for layer in cfg.model_spec().layers)


def test_registry_resolves_and_refuses(tmp_path):
    assert "Qwen3ForCausalLM" in supported_architectures()
    with pytest.raises(ValueError, match="unsupported architecture 'LlamaForCausalLM'"):
        resolve_config({**plain.TINY_A, "architectures": ["LlamaForCausalLM"]})
    no_arch = {k: v for k, v in plain.TINY_A.items() if k != "architectures"}
    assert isinstance(resolve_config(no_arch), Qwen3Config)     # falls back on model_type
    with pytest.raises(ValueError, match="names no architecture"):
        resolve_config({"hidden_size": 8})
    (tmp_path / "config.json").write_text(json.dumps(plain.TINY_C))
    assert load_config(str(tmp_path)).head_dim == 48
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path / "nothing"))


def test_a_new_architecture_registers_without_touching_the_framework():
    class ToyConfig(ModelConfig):
        architecture = "ToyForCausalLM"

        def __init__(self, data):
            self.data = data

        @classmethod
        def from_json(cls, data):
            return cls(data)

    register_architecture("ToyForCausalLM", ToyConfig)
    cfg = resolve_config({"architectures": ["ToyForCausalLM"], "x": 1})
    assert isinstance(cfg, ToyConfig) and cfg.data["x"] == 1
    with pytest.raises(TypeError):
        register_architecture("Bad", dict)


def test_parameter_count_matches_tensor_shapes():
    for tiny in (plain.TINY_A, plain.TINY_B, plain.TINY_C):
        total = sum(int(__import__("math").prod(s)) for s in plain.tensor_shapes(tiny).values())
        assert resolve_config(tiny).parameter_counts()["total_parameters"] == total
