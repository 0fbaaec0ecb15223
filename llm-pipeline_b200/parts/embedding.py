"""Token embedding (src/llm_pipeline/models/qwen3/custom_builder.py:300-305,323: a plain row
gather) and the output head (:387-391,415: a bias-free linear layer whose weight is the embedding
table when ``tie_word_embeddings`` is set). The head returns float32 logits."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .base import Embedding, Head, TensorGetter
from .registry import register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int):
        self.prefix, self.vocab_size, self.hidden_size = prefix, int(vocab_size), int(hidden_size)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {f"{self.prefix}.weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, get: TensorGetter) -> None:
        self.weight = get(f"{self.prefix}.weight", "matrix").contiguous()

    def forward(self, ctx) -> torch.Tensor:
        out = torch.empty((ctx.num_tokens, self.hidden_size), dtype=torch.float32, device=ctx.device)
        kernels.embedding(ctx.token_ids, self.weight, out)
        return out


@register_head("linear_head")
class LinearHead(Head):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None):
        self.prefix, self.vocab_size, self.hidden_size, self.tied_to = prefix, int(vocab_size), int(hidden_size), tied_to
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        # A tied head has no tensor of its own; a checkpoint may still carry a copy, which must be one.
        return {f"{self.prefix}.weight": ParamSpec((self.vocab_size, self.hidden_size), optional=self.tied_to is not None)}

    def copies(self) -> Dict[str, str]:
        # The reference makes the head's parameter the embedding's own tensor when tie_word_embeddings is set
        # (models/qwen3/custom_builder.py:389-391), so a checkpoint it wrote holds the same values under both names.
        return {f"{self.prefix}.weight": f"{self.tied_to}.weight"} if self.tied_to else {}

    def load(self, get: TensorGetter) -> None:
        name = f"{self.tied_to}.weight" if self.tied_to else f"{self.prefix}.weight"
        self.weight = get(name, "matrix")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return linear(x, self.weight, out_dtype=torch.float32)
