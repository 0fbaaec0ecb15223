"""Where tensors come from: a folder of safetensors files, a dictionary, or a seeded generator.

The reference iterates every ``*.safetensors`` file of the model folder and copies each tensor
into the parameter of the same name (src/llm_pipeline/models/qwen3/custom_loader.py:15-32); a
missing tensor is left at its initial value without a word and an unknown name raises from
``get_parameter``. Here names and shapes are checked as a whole before anything is copied, and
one ``WeightError`` lists every missing tensor, unexpected tensor and wrong shape.
"""

from __future__ import annotations

import glob
import hashlib
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch


class WeightError(ValueError):
    """The checkpoint does not match the model. ``missing``, ``unexpected`` and ``wrong_shape``
    hold the tensor names of each kind."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[Tuple[str, tuple, tuple]]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = ["the checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        super().__init__("\n".join(lines))


class TiedWeightError(ValueError):
    """The checkpoint holds a tensor that the model reads under another name, with other values."""

    def __init__(self, name: str, original: str):
        self.name, self.original = name, original
        super().__init__(f"the checkpoint's {name} differs from {original}, which the model uses in its place "
                         f"(tied weights): one of the two is not what the configuration says")


@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part expects. ``role``: "matrix" (operand of a matrix product, kept in the
    compute type), "vector" (norm weight or bias: kept in float32 when stored so, else in the
    compute type), "table" (integers, kept as int32). ``optional`` tensors may be absent;
    ``init`` tells the random-weights mode how to draw it ("normal" or "norm")."""

    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
    init: str = "normal"


# Names a checkpoint may hold that are no parameters (the rotary table is recomputed).
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightSource:
    def names(self) -> List[str]:
        raise NotImplementedError

    def shape(self, name: str) -> Tuple[int, ...]:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        """The tensor as stored (CPU unless the source generates on a device)."""
        raise NotImplementedError


class DictSource(WeightSource):
    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.tensors = tensors

    def names(self):
        return list(self.tensors)

    def shape(self, name):
        return tuple(self.tensors[name].shape)

    def get(self, name):
        return self.tensors[name]


class SafetensorsSource(WeightSource):
    """All ``*.safetensors`` files of a folder, addressed by tensor name."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open

        self.files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
        if not self.files:
            raise FileNotFoundError(f"no *.safetensors file in {model_dir!r}")
        self._open = safe_open
        self._where: Dict[str, str] = {}
        self._shapes: Dict[str, Tuple[int, ...]] = {}
        duplicates = []
        for path in self.files:
            with safe_open(path, "pt", "cpu") as f:
                for name in f.keys():
                    if name in self._where:
                        duplicates.append(name)
                    self._where[name] = path
                    self._shapes[name] = tuple(f.get_slice(name).get_shape())
        if duplicates:
            raise WeightError([], [f"{n} (stored twice)" for n in duplicates], [])
        self._handles: Dict[str, object] = {}

    def names(self):
        return list(self._where)

    def shape(self, name):
        return self._shapes[name]

    def get(self, name):
        path = self._where[name]
        handle = self._handles.get(path)
        if handle is None:
            handle = self._open(path, "pt", "cpu")
            handle.__enter__()
            self._handles[path] = handle
        return handle.get_tensor(name)

    def close(self):
        for handle in self._handles.values():
            handle.__exit__(None, None, None)
        self._handles.clear()


class RandomSource(WeightSource):
    """Seeded random tensors for the expected parameters: matrices N(0, std), norm weights
    1 + N(0, 0.1), drawn in float32 and rounded to ``dtype``. Every tensor has a generator of its
    own, seeded from (seed, name), so a tensor's values do not depend on which others are drawn."""

    def __init__(self, expected: Dict[str, ParamSpec], seed: int, std: float = 0.02,
                 dtype: torch.dtype = torch.bfloat16, device: str = "cpu"):
        self.expected = {n: s for n, s in expected.items() if not s.optional}
        self.seed, self.std, self.dtype, self.device = int(seed), float(std), dtype, torch.device(device)

    def names(self):
        return list(self.expected)

    def shape(self, name):
        return tuple(self.expected[name].shape)

    def get(self, name):
        spec = self.expected[name]
        digest = hashlib.sha256(f"{self.seed}:{name}".encode()).digest()
        gen = torch.Generator(device=self.device).manual_seed(int.from_bytes(digest[:8], "little") >> 1)
        if spec.role == "table":
            return torch.zeros(spec.shape, dtype=torch.int32, device=self.device)
        noise = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=self.device)
        value = noise.mul_(0.1).add_(1.0) if spec.init == "norm" else noise.mul_(self.std)
        return value.to(self.dtype)


def check_names_and_shapes(expected: Dict[str, ParamSpec], source: WeightSource,
                           ignorable: Iterable[str] = ()) -> None:
    """Raise one ``WeightError`` that lists all missing, unexpected and mis-shaped tensors."""
    have = set(source.names())
    ignorable = set(ignorable)
    missing = [n for n, s in expected.items() if n not in have and not s.optional]
    unexpected = sorted(n for n in have if n not in expected and n not in ignorable
                        and not n.endswith(IGNORED_SUFFIXES))
    wrong = [(n, source.shape(n), tuple(s.shape)) for n, s in expected.items()
             if n in have and tuple(source.shape(n)) != tuple(s.shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)


def stored_dtype_policy(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The type a tensor is kept in on the device: integer tables as int32; with a float32
    compute type everything is float32; otherwise matrices take the compute type (bfloat16) and a
    vector that was stored in 32-bit stays so."""
    if role == "table" or not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if role == "vector" and stored == torch.float32:
        return torch.float32
    return compute
