"""Typed configuration of the Qwen3 dense decoder, read from its ``config.json`` keys.

The keys and their fall-backs follow DavidAkinpelu/llm-pipeline:
src/llm_pipeline/models/qwen3/config.py:49-88 (key names and aliases) and
src/llm_pipeline/models/qwen3/custom_builder.py:30-42,68 (defaults the model code applies:
``rms_norm_eps`` 1e-6, ``attention_bias`` False, ``rope_theta`` 1000000, ``head_dim`` falling
back to ``hidden_size // num_attention_heads``).

Three keys are read and, as in the reference's model code, have no effect on the result; a
warning says so when they ask for something else: ``rope_scaling`` (custom_builder.py:263 fixes
the default rotary type), ``use_sliding_window``/``sliding_window`` (custom_builder.py:154-160
always builds the full causal mask) and ``hidden_act`` (custom_builder.py:204 fixes SiLU).
"""

from __future__ import annotations

import warnings
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Union

from .base import LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

_REQUIRED = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "intermediate_size")


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    head_dim: int
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    attention_bias: bool = False
    attention_dropout: float = 0.0
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    tie_word_embeddings: bool = False
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Union[None, int, List[int]] = None
    torch_dtype: str = "bfloat16"
    model_type: str = "qwen3"

    architecture = "Qwen3ForCausalLM"

    # reference aliases (src/llm_pipeline/models/qwen3/config.py:90-97)
    @property
    def num_layers(self) -> int:
        return self.num_hidden_layers

    @property
    def norm_epsilon(self) -> float:
        return self.rms_norm_eps

    @property
    def num_key_value_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "Qwen3Config":
        def first(*names, default=None):
            for name in names:
                if data.get(name) is not None:
                    return data[name]
            return default

        d = dict(data)
        if d.get("num_hidden_layers") is None and d.get("num_layers") is not None:
            d["num_hidden_layers"] = d["num_layers"]
        missing = [k for k in _REQUIRED if d.get(k) is None]
        if missing:
            raise ValueError(f"Qwen3 config.json lacks required keys: {missing}")
        hidden, heads = int(d["hidden_size"]), int(d["num_attention_heads"])
        head_dim = first("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ValueError("config.json has no head_dim and hidden_size is not a multiple of "
                                 "num_attention_heads")
            head_dim = hidden // heads
        nested = d.get("rope_parameters") or {}
        rope_theta = first("rope_theta", "default_theta")
        if rope_theta is None:
            rope_theta = nested.get("rope_theta", 1000000.0)
        rope_scaling = d.get("rope_scaling")
        if rope_scaling is None and nested.get("rope_type", "default") != "default":
            rope_scaling = dict(nested)
        config = cls(
            vocab_size=int(d["vocab_size"]), hidden_size=hidden,
            num_hidden_layers=int(d["num_hidden_layers"]), num_attention_heads=heads,
            num_key_value_heads=int(d["num_key_value_heads"]),
            intermediate_size=int(d["intermediate_size"]), head_dim=int(head_dim),
            max_position_embeddings=int(first("max_position_embeddings", default=32768)),
            rms_norm_eps=float(first("rms_norm_eps", "norm_epsilon", default=1e-6)),
            rope_theta=float(rope_theta), rope_scaling=rope_scaling,
            attention_bias=bool(first("attention_bias", default=False)),
            attention_dropout=float(first("attention_dropout", default=0.0)),
            hidden_act=str(first("hidden_act", default="silu")),
            use_sliding_window=bool(first("use_sliding_window", default=False)),
            sliding_window=first("sliding_window", "sliding_window_size"),
            tie_word_embeddings=bool(first("tie_word_embeddings", default=False)),
            pad_token_id=d.get("pad_token_id"), bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id"),
            torch_dtype=str(first("dtype", "torch_dtype", default="bfloat16")),
            model_type=str(first("model_type", default="qwen3")),
        )
        config.validate()
        return config

    def validate(self) -> None:
        problems = []
        for name in _REQUIRED + ("head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                problems.append(f"{name} must be positive, got {getattr(self, name)}")
        if not problems:
            if self.num_attention_heads % self.num_key_value_heads:
                problems.append(f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                                f"num_key_value_heads ({self.num_key_value_heads})")
            if self.head_dim % 2:
                problems.append(f"head_dim ({self.head_dim}) must be even for the rotary encoding")
        if not self.rms_norm_eps > 0:
            problems.append(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            problems.append(f"rope_theta must be positive, got {self.rope_theta}")
        if self.model_type != "qwen3":
            problems.append(f"model_type is {self.model_type!r}, expected 'qwen3'")
        if problems:
            raise ValueError("invalid Qwen3 configuration: " + "; ".join(problems))
        if self.rope_scaling and str(self.rope_scaling.get("rope_type", self.rope_scaling.get("type", "default"))) != "default":
            warnings.warn("rope_scaling is set, but the Qwen3 dense model applies the default rotary "
                          "encoding only; the key has no effect", stacklevel=2)
        if self.use_sliding_window:
            warnings.warn("use_sliding_window is set, but the Qwen3 dense model attends to all earlier "
                          "tokens; the key has no effect", stacklevel=2)
        if self.hidden_act != "silu":
            warnings.warn(f"hidden_act is {self.hidden_act!r}, but the Qwen3 dense feed-forward always "
                          "uses SiLU; the key has no effect", stacklevel=2)

    def to_json(self) -> Dict[str, Any]:
        out = asdict(self)
        out["architectures"] = [self.architecture]
        return out

    def eos_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, (list, tuple)):
            return [int(t) for t in self.eos_token_id]
        return [int(self.eos_token_id)]

    def parameter_counts(self) -> Dict[str, int]:
        """Closed form of src/llm_pipeline/models/qwen3/factory.py:32-75."""
        attention = self.hidden_size * (self.q_size + 2 * self.kv_size) + self.q_size * self.hidden_size
        if self.attention_bias:
            attention += self.q_size + 2 * self.kv_size + self.hidden_size
        per_layer = attention + 2 * self.head_dim + 3 * self.hidden_size * self.intermediate_size + 2 * self.hidden_size
        embedding = self.vocab_size * self.hidden_size
        head = 0 if self.tie_word_embeddings else embedding
        return {"embedding_parameters": embedding, "parameters_per_layer": per_layer,
                "final_norm_parameters": self.hidden_size, "lm_head_parameters": head,
                "total_parameters": embedding + per_layer * self.num_hidden_layers + self.hidden_size + head}

    def model_spec(self) -> ModelSpec:
        """The layer list of src/llm_pipeline/models/qwen3/custom_builder.py:210-255,291-375: every
        layer is a pre-norm residual block of grouped-query attention with per-head q/k RMSNorm and
        rotary positions, and a SwiGLU feed-forward; embedding before, RMSNorm and output head after."""
        norm = {"size": self.hidden_size, "eps": self.rms_norm_eps}
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}"
            layers.append(LayerSpec(
                block="pre_norm_residual",
                mixer=PartSpec("attention", {
                    "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                    "bias": self.attention_bias, "qk_norm": True, "qk_norm_eps": self.rms_norm_eps,
                    "scale": self.head_dim ** -0.5, "window": None, "position": "rope",
                }, f"{p}.self_attn"),
                feed_forward=PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                                 "intermediate_size": self.intermediate_size}, f"{p}.mlp"),
                mixer_norm=PartSpec("rms_norm", dict(norm), f"{p}.input_layernorm"),
                feed_forward_norm=PartSpec("rms_norm", dict(norm), f"{p}.post_attention_layernorm"),
            ))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size},
                               "model.embed_tokens"),
            positions={"rope": PartSpec("rotary", {"rotary_dim": self.head_dim, "theta": self.rope_theta,
                                                   "scaling": 1.0})},
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rms_norm", dict(norm), "model.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                          "tied_to": "model.embed_tokens" if self.tie_word_embeddings else None},
                          "lm_head"),
            max_position=self.max_position_embeddings,
        )
        spec.validate()
        return spec


register_architecture("Qwen3ForCausalLM", Qwen3Config)
