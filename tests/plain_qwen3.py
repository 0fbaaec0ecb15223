"""Plain, slow Qwen3 dense decoder used as the oracle by the tests.

Whole sequences, no cache, one function per part, float32 (or float64) on
whatever device the tensors live on. It shares no code with the engine: it reads
a ``config.json`` dict and a ``{tensor name: tensor}`` dict directly.

Every function restates a formula of DavidAkinpelu/llm-pipeline and cites it as
``src/llm_pipeline/<file>:<lines>``. ``tests/golden/make_golden.py`` compares this
file once with the reference's own ``Qwen3ForCausalLM`` on the CPU.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def cfg_get(config: dict, key: str, default=None):
    value = config.get(key, default)
    return default if value is None else value


def head_dim_of(config: dict) -> int:
    # models/qwen3/custom_builder.py:68 — head_dim, else hidden_size // num_attention_heads
    return int(cfg_get(config, "head_dim", config["hidden_size"] // config["num_attention_heads"]))


def rope_theta_of(config: dict) -> float:
    # models/qwen3/custom_builder.py:41-42 — default 1000000 when the key is absent
    if config.get("rope_theta") is not None:
        return float(config["rope_theta"])
    nested = config.get("rope_parameters") or {}
    if nested.get("rope_theta") is not None:
        return float(nested["rope_theta"])
    return 1000000.0


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """models/qwen3/custom_builder.py:53-58 — w * (x * rsqrt(mean(x^2) + eps))."""
    variance = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    """models/qwen3/custom_builder.py:269-288 — inv_freq = 1/theta^(2j/d); angles = pos * inv_freq;
    cos/sin of cat(angles, angles). The frequency table and the angles are float32 there."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
    inv_freq = (1.0 / (theta ** exponent)).to(positions.device)
    freqs = positions.float()[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """models/qwen3/custom_builder.py:85-89 — cat(-x2, x1)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """models/qwen3/custom_builder.py:91-99 — x*cos + rotate_half(x)*sin; x is [heads, T, d]."""
    return x * cos[None] + rotate_half(x) * sin[None]


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ weight.t()
    return y if bias is None else y + bias


def attention(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, config: dict,
              cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """models/qwen3/custom_builder.py:110-190 for one whole sequence x [T, H] and no past."""
    T = x.shape[0]
    d = head_dim_of(config)
    nq = config["num_attention_heads"]
    nkv = config["num_key_value_heads"]
    eps = float(cfg_get(config, "rms_norm_eps", 1e-6))
    bias = bool(cfg_get(config, "attention_bias", False))

    def proj(name):
        return linear(x, w[f"{prefix}.{name}.weight"], w[f"{prefix}.{name}.bias"] if bias else None)

    # :124-126 — project, split into heads [heads, T, d]
    q = proj("q_proj").view(T, nq, d).transpose(0, 1)
    k = proj("k_proj").view(T, nkv, d).transpose(0, 1)
    v = proj("v_proj").view(T, nkv, d).transpose(0, 1)
    # :129-130 — per-head RMSNorm over d, one weight for all heads
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    # :133-134 — rotary on q and k
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    # :101-108,144-145 — each kv head serves nq // nkv consecutive query heads
    group = nq // nkv
    k = k.repeat_interleave(group, dim=0)
    v = v.repeat_interleave(group, dim=0)
    # :148 — scores scaled by d^-0.5 after the product
    scores = (q @ k.transpose(1, 2)) * (d ** -0.5)
    # :154-160 — causal: key position > query position is masked
    pos = torch.arange(T, device=x.device)
    masked = pos[None, :] > pos[:, None]
    scores = scores.masked_fill(masked[None], float("-inf"))
    # :179 — softmax in float32
    probs = torch.softmax(scores, dim=-1)
    # :183-188 — weighted sum, heads back to columns, output projection
    out = (probs @ v).transpose(0, 1).reshape(T, nq * d)
    return linear(out, w[f"{prefix}.o_proj.weight"], w[f"{prefix}.o_proj.bias"] if bias else None)


def mlp(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """models/qwen3/custom_builder.py:206-207 — down(silu(gate(x)) * up(x)), no biases."""
    gate = linear(x, w[f"{prefix}.gate_proj.weight"])
    up = linear(x, w[f"{prefix}.up_proj.weight"])
    return linear(torch.nn.functional.silu(gate) * up, w[f"{prefix}.down_proj.weight"])


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], index: int, config: dict,
                  cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """models/qwen3/custom_builder.py:222-255 — two pre-norm residual halves."""
    eps = float(cfg_get(config, "rms_norm_eps", 1e-6))
    prefix = f"model.layers.{index}"
    h = rms_norm(x, w[f"{prefix}.input_layernorm.weight"], eps)
    x = x + attention(h, w, f"{prefix}.self_attn", config, cos, sin)
    h = rms_norm(x, w[f"{prefix}.post_attention_layernorm.weight"], eps)
    return x + mlp(h, w, f"{prefix}.mlp")


def forward_logits(config: dict, weights: Dict[str, torch.Tensor], token_ids: Sequence[int],
                   dtype: torch.dtype = torch.float32, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """models/qwen3/custom_builder.py:311-375,393-421 — logits [T, V] of one whole sequence. ``rows`` keeps only
    those positions for the output head (a large vocabulary times a long sequence is a lot of logits nobody reads);
    the layers always run on the whole sequence."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    device = next(iter(w.values())).device
    ids = torch.as_tensor(list(token_ids), dtype=torch.long, device=device)
    x = w["model.embed_tokens.weight"][ids]                                   # :323
    positions = torch.arange(len(ids), device=device)                           # :332-337
    cos, sin = rope_cos_sin(positions, head_dim_of(config), rope_theta_of(config))
    cos, sin = cos.to(dtype), sin.to(dtype)                                     # :288
    for index in range(config["num_hidden_layers"]):                            # :353-368
        x = decoder_layer(x, w, index, config, cos, sin)
    x = rms_norm(x, w["model.norm.weight"], float(cfg_get(config, "rms_norm_eps", 1e-6)))  # :370
    if bool(cfg_get(config, "tie_word_embeddings", False)):                     # :389-391
        head = w["model.embed_tokens.weight"]
    else:
        head = w["lm_head.weight"]
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long, device=device)]
    return x @ head.t()                                                         # :415


def greedy_generate(config: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int],
                    max_new_tokens: int, eos_token_id: Optional[int] = None) -> List[int]:
    """models/qwen3/custom_builder.py:423-509 with do_sample False, recomputing the whole
    sequence for every token (no cache)."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(max_new_tokens):
        token = int(torch.argmax(forward_logits(config, weights, ids)[-1]).item())
        out.append(token)
        ids.append(token)
        if eos_token_id is not None and token == eos_token_id:
            break
    return out


# --------------------------------------------------------------------------------------
# Sampler (inference/sampling.py). Filters return logits with -inf at removed entries.
# --------------------------------------------------------------------------------------

def apply_repetition_penalty(logits: torch.Tensor, generated: Sequence[int], penalty: float) -> torch.Tensor:
    """inference/sampling.py:108-137 — positive logits divided, others multiplied, once per token id."""
    if not generated or penalty == 1.0:
        return logits
    out = logits.clone()
    for token in set(int(t) for t in generated):
        if 0 <= token < logits.shape[-1]:
            value = out[..., token]
            out[..., token] = torch.where(value > 0, value / penalty, value * penalty)
    return out


def apply_top_k(logits: torch.Tensor, top_k: int) -> torch.Tensor:
    """inference/sampling.py:139-156 — keep logits >= the k-th largest."""
    if top_k <= 0:
        return logits
    k = min(top_k, logits.shape[-1])
    kth = torch.topk(logits, k, dim=-1).values[..., -1:]
    return torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)


def apply_top_p(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    """inference/sampling.py:158-185 — sort descending; drop a token when the mass before it exceeds p."""
    if top_p >= 1.0:
        return logits
    sorted_logits, order = torch.sort(logits, descending=True, dim=-1)
    cumulative = torch.cumsum(torch.softmax(sorted_logits, dim=-1), dim=-1)
    remove = cumulative > top_p
    remove[..., 1:] = remove[..., :-1].clone()
    remove[..., 0] = False
    mask = torch.zeros_like(remove).scatter(-1, order, remove)
    return logits.masked_fill(mask, float("-inf"))


def apply_min_p(logits: torch.Tensor, min_p: float) -> torch.Tensor:
    """inference/sampling.py:187-205 — drop prob < min_p * max prob."""
    if min_p <= 0.0:
        return logits
    probs = torch.softmax(logits, dim=-1)
    return logits.masked_fill(probs < min_p * probs.max(dim=-1, keepdim=True).values, float("-inf"))


def apply_typical_p(logits: torch.Tensor, typical_p: float) -> torch.Tensor:
    """inference/sampling.py:207-238 — keep -log p <= exp(entropy) * typical_p, else the argmax."""
    if typical_p >= 1.0:
        return logits
    log_probs = torch.log_softmax(logits, dim=-1)
    probs = log_probs.exp()
    entropy = -(probs * torch.where(probs > 0, log_probs, torch.zeros_like(log_probs))).sum(-1, keepdim=True)
    keep = (-log_probs) <= torch.exp(entropy) * typical_p
    empty = ~keep.any(dim=-1)
    if empty.any():
        keep[empty, logits[empty].argmax(dim=-1)] = True
    return torch.where(keep, logits, torch.full_like(logits, float("-inf")))


def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0,
                   min_p: float = 0.0, typical_p: float = 1.0, repetition_penalty: float = 1.0,
                   generated: Sequence[int] = ()) -> torch.Tensor:
    """inference/sampling.py:69-84 — the order of the filters, then softmax. temperature must be > 0."""
    logits = apply_repetition_penalty(logits.float(), generated, repetition_penalty)
    logits = logits / temperature
    logits = apply_top_k(logits, top_k)
    logits = apply_top_p(logits, top_p)
    logits = apply_min_p(logits, min_p)
    logits = apply_typical_p(logits, typical_p)
    return torch.softmax(logits, dim=-1)


def inverse_cdf_pick(probs: torch.Tensor, u: float) -> int:
    """The draw the engine documents: the first index whose running sum of probabilities exceeds
    u * total (the reference draws with torch.multinomial from the global generator instead,
    inference/sampling.py:85)."""
    cdf = torch.cumsum(probs.double(), dim=-1)
    target = u * float(cdf[-1])
    return int(min(int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype), right=True)),
                   probs.shape[-1] - 1))


# --------------------------------------------------------------------------------------
# Random weights in the reference's tensor names (used by tests that need a model folder)
# --------------------------------------------------------------------------------------

def tensor_shapes(config: dict) -> Dict[str, tuple]:
    """Names and shapes of models/qwen3/custom_builder.py's module tree (:68-83,197-203,300-307,387-391)."""
    H = config["hidden_size"]
    d = head_dim_of(config)
    nq, nkv = config["num_attention_heads"], config["num_key_value_heads"]
    I, V = config["intermediate_size"], config["vocab_size"]
    shapes: Dict[str, tuple] = {"model.embed_tokens.weight": (V, H)}
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}"
        shapes[f"{p}.input_layernorm.weight"] = (H,)
        shapes[f"{p}.self_attn.q_proj.weight"] = (nq * d, H)
        shapes[f"{p}.self_attn.k_proj.weight"] = (nkv * d, H)
        shapes[f"{p}.self_attn.v_proj.weight"] = (nkv * d, H)
        shapes[f"{p}.self_attn.o_proj.weight"] = (H, nq * d)
        if cfg_get(config, "attention_bias", False):
            shapes[f"{p}.self_attn.q_proj.bias"] = (nq * d,)
            shapes[f"{p}.self_attn.k_proj.bias"] = (nkv * d,)
            shapes[f"{p}.self_attn.v_proj.bias"] = (nkv * d,)
            shapes[f"{p}.self_attn.o_proj.bias"] = (H,)
        shapes[f"{p}.self_attn.q_norm.weight"] = (d,)
        shapes[f"{p}.self_attn.k_norm.weight"] = (d,)
        shapes[f"{p}.post_attention_layernorm.weight"] = (H,)
        shapes[f"{p}.mlp.gate_proj.weight"] = (I, H)
        shapes[f"{p}.mlp.up_proj.weight"] = (I, H)
        shapes[f"{p}.mlp.down_proj.weight"] = (H, I)
    shapes["model.norm.weight"] = (H,)
    if not cfg_get(config, "tie_word_embeddings", False):
        shapes["lm_head.weight"] = (V, H)
    return shapes


def random_weights(config: dict, seed: int, std: float = 0.02, dtype: torch.dtype = torch.float32,
                   ) -> Dict[str, torch.Tensor]:
    """Matrices N(0, std), norm weights 1 + N(0, 0.1), biases N(0, std); drawn in name order."""
    gen = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(config).items():
        noise = torch.randn(shape, generator=gen, dtype=torch.float32)
        if "norm" in name:
            value = 1.0 + 0.1 * noise
        else:
            value = std * noise
        out[name] = value.to(dtype)
    return out


TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "attention_bias": False,
    "max_position_embeddings": 512, "hidden_act": "silu",
}

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 224, "vocab_size": 384, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 1024, "hidden_act": "silu",
}

# A third shape: biases on, head_dim 48 (a multiple of 16 that is no power of two), 3 groups of 3.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 9, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 176, "vocab_size": 331, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "attention_bias": True,
    "max_position_embeddings": 2048, "hidden_act": "silu",
}

# A fourth shape: head_dim 128 (the size that the tcgen05 prefill attention kernel takes in bfloat16), groups of 2.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 160, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 288, "vocab_size": 300, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 2048, "hidden_act": "silu",
}

# widths in multiples of 64, which the streaming products of a decode step take: the norm between two of them is then
# folded into them
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 2, "num_key_value_heads": 1,
    "head_dim": 64, "intermediate_size": 192, "vocab_size": 211, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "attention_bias": False,
    "max_position_embeddings": 1024, "hidden_act": "silu",
}
