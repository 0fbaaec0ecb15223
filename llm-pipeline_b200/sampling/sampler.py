"""Token selection: greedy and temperature sampling with the reference's filters.

Names, defaults and order follow src/llm_pipeline/inference/sampling.py:10-37,51-85:
repetition penalty, then ``logits / temperature`` (``temperature <= 0`` means argmax), top-k,
top-p, min-p, typical-p, softmax and one draw. ``do_sample`` is carried and, as there
(:67-85), never read. The work is done by one CUDA kernel per batch (``csrc/sampling.cu``); the
draw is an inverse-CDF pick with a uniform number from a counter-based generator keyed by the
request's ``seed`` and its count of sampled tokens, so a request's tokens do not depend on what
else is in the batch (the reference draws with ``torch.multinomial`` from the global generator,
:85). Mirostat v2 (:240-279), which the reference's sampler offers and its engine never calls, is
``sample_mirostat_v2`` here, with the same arithmetic.

Typical-p: the reference's entropy is NaN as soon as an earlier filter has removed a token
(0 * -inf at :226), which leaves only the most likely token; here the entropy is taken over the
tokens that are still kept.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass, replace
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..ops import kernels


@dataclass
class SamplingConfig:
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    typical_p: float = 1.0
    min_p: float = 0.0
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    do_sample: bool = True
    pad_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    seed: int = 0

    def merged(self, override: Optional[Dict[str, Any]]) -> "SamplingConfig":
        if not override:
            return self
        known = {k: v for k, v in override.items() if k in self.__dataclass_fields__ and v is not None}
        return replace(self, **known)


def _f2i(value: float) -> int:
    return struct.unpack("<i", struct.pack("<f", float(value)))[0]


def _u2i(value: int) -> int:
    value &= 0xFFFFFFFF
    return value - (1 << 32) if value >= (1 << 31) else value


def pack_rows(configs: Sequence[SamplingConfig], steps: Sequence[int]) -> torch.Tensor:
    """int32 [rows, 8]: temperature, top_k, top_p, min_p, typical_p (floats by bit pattern),
    seed low, seed high, step."""
    rows = []
    for cfg, step in zip(configs, steps):
        seed = int(cfg.seed) & 0xFFFFFFFFFFFFFFFF
        rows.append([_f2i(cfg.temperature), int(cfg.top_k), _f2i(cfg.top_p), _f2i(cfg.min_p), _f2i(cfg.typical_p),
                     _u2i(seed), _u2i(seed >> 32), _u2i(int(step))])
    return torch.tensor(rows, dtype=torch.int32)


def uniform_of(seed: int, step: int) -> float:
    """The uniform number in [0, 1) that row (seed, step) draws with (24 bits of Philox4x32-10)."""
    import ctypes

    from ..ops import library

    fn = library().llmp_philox_first
    fn.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong]
    fn.restype = ctypes.c_uint
    return (fn(int(seed) & 0xFFFFFFFFFFFFFFFF, int(step)) >> 8) / 16777216.0


class Sampler:
    def __init__(self, config: Optional[SamplingConfig] = None):
        self.config = config or SamplingConfig()

    def sample_rows(self, logits: torch.Tensor, configs: Sequence[SamplingConfig], steps: Sequence[int],
                    generated: Optional[Sequence[Optional[Sequence[int]]]] = None) -> torch.Tensor:
        """One token per row of float32 ``logits [rows, vocab]`` on a CUDA device, each row with its
        own parameters; ``steps[i]`` is how many tokens row i's request has sampled before;
        ``generated[i]`` are the tokens a repetition penalty applies to. Returns int32 ``[rows]``."""
        if logits.dim() != 2 or logits.dtype != torch.float32 or not logits.is_cuda:
            raise kernels.KernelError("sampling takes float32 logits [rows, vocab] on a CUDA device")
        M = logits.shape[0]
        out = torch.empty(M, dtype=torch.int32, device=logits.device)
        if M == 0:
            return out
        if all(not c.temperature > 0 for c in configs) and not any(c.repetition_penalty != 1.0 for c in configs):
            return kernels.argmax(logits, out)
        if generated is not None and any(c.repetition_penalty != 1.0 and g for c, g in zip(configs, generated)):
            tokens: List[int] = []
            offsets = [0]
            for cfg, g in zip(configs, generated):
                if g and cfg.repetition_penalty != 1.0:
                    tokens.extend(sorted(set(int(t) for t in g)))
                offsets.append(len(tokens))
            logits = logits.clone()
            dev = logits.device
            kernels.repetition_penalty(
                logits, torch.tensor(tokens or [0], dtype=torch.int32, device=dev),
                torch.tensor(offsets, dtype=torch.int32, device=dev),
                torch.tensor([c.repetition_penalty for c in configs], dtype=torch.float32, device=dev))
        params = pack_rows(configs, steps).to(logits.device)
        return kernels.sample(logits, params, out)

    def sample_token(self, logits: torch.Tensor, config_override: Optional[Dict[str, Any]] = None,
                     generated_tokens: Optional[List[int]] = None, step: int = 0) -> torch.Tensor:
        """The reference's call: one configuration for all rows of ``logits [batch, vocab]``; returns
        token ids ``[batch]`` (int64). Row i draws with seed ``seed + i``."""
        cfg = self.config.merged(config_override)
        rows = [replace(cfg, seed=cfg.seed + i) for i in range(logits.shape[0])]
        out = self.sample_rows(logits.float().contiguous(), rows, [step] * logits.shape[0],
                               [generated_tokens] * logits.shape[0])
        return out.long()

    def sample_mirostat_v2(self, logits: torch.Tensor, config_override: Optional[Dict[str, Any]] = None,
                           previous_entropy: Optional[float] = None, step: int = 0):
        """Mirostat v2 as in src/llm_pipeline/inference/sampling.py:240-279, for one row of ``logits [1, vocab]``: the
        entropy H of softmax(logits / temperature); ``previous_entropy`` (H itself at the first call) moves by
        ``-mirostat_eta * (H - mirostat_tau)``; while it is positive the draw is among the ``int(exp(previous_entropy))``
        most likely tokens (at least one), else among all. Returns (token ids ``[1]`` int64, the new value to pass in
        at the next call). The entropy and the draw are this library's kernels; the draw uses the request's seed and
        ``step`` like every other draw here (the reference draws with ``torch.multinomial``, :277)."""
        import math
        cfg = self.config.merged(config_override)
        if logits.dim() != 2 or logits.shape[0] != 1:
            raise ValueError("Mirostat steers one sequence: logits must be [1, vocab] (the reference reads the entropy "
                             "with .item(), :266-269)")
        logits = logits.float().contiguous()
        current = float(kernels.entropy(logits, cfg.temperature)[0])
        if previous_entropy is None:
            previous_entropy = current
        previous_entropy -= cfg.mirostat_eta * (current - cfg.mirostat_tau)
        top_k = max(1, int(math.exp(previous_entropy))) if previous_entropy > 0 else 0
        draw = replace(cfg, temperature=cfg.temperature if cfg.temperature > 0 else 1.0, top_k=min(top_k, logits.shape[1]),
                       top_p=1.0, min_p=0.0, typical_p=1.0, repetition_penalty=1.0)
        out = self.sample_rows(logits, [draw], [step], None)
        return out.long(), previous_entropy

    def get_sampling_info(self) -> Dict[str, Any]:
        c = self.config
        return {"temperature": c.temperature, "top_k": c.top_k, "top_p": c.top_p,
                "repetition_penalty": c.repetition_penalty, "typical_p": c.typical_p, "min_p": c.min_p,
                "mirostat_tau": c.mirostat_tau, "mirostat_eta": c.mirostat_eta, "do_sample": c.do_sample}
