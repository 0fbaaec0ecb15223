"""Architecture-neutral description of a model: which parts, with which sizes, in which order.

A typed configuration (one class per architecture, see ``qwen3.py``) reads the architecture's own
``config.json`` keys and turns them into a ``ModelSpec``. Everything below the configuration
(parts, cache manager, step function, scheduler, replay) works from the ``ModelSpec`` alone, so a
new architecture is a new configuration class plus, where needed, new part kinds.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` is the key in the part registry, ``args`` are its sizes and constants,
    ``prefix`` is the prefix of its tensor names in the checkpoint."""

    kind: str
    args: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of a mixer, a feed-forward and their norms.
    Different layers of one model may name different kinds. A block finds its norms by name:
    ``mixer_norm`` and ``feed_forward_norm`` are the two of a pre-norm block (names "mixer" and
    "feed_forward"); ``norms`` holds any further ones a block kind asks for (post-norms, a norm
    of a parallel branch, ...), so a block with four norms or with none is a matter of
    configuration."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    norms: Dict[str, PartSpec] = field(default_factory=dict)

    def named_norms(self) -> Dict[str, PartSpec]:
        out: Dict[str, PartSpec] = {}
        if self.mixer_norm is not None:
            out["mixer"] = self.mixer_norm
        if self.feed_forward_norm is not None:
            out["feed_forward"] = self.feed_forward_norm
        for name, spec in self.norms.items():
            if name in out:
                raise ValueError(f"the layer names its norm {name!r} twice")
            out[name] = spec
        return out


@dataclass(frozen=True)
class ScheduleEntry:
    """One executed layer. ``layer`` indexes ``ModelSpec.layers`` (the same layer may appear
    twice); ``cache`` is the id of the cache this execution uses. The first entry that names a
    cache id writes it, a later entry with the same id only reads it."""

    layer: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartSpec
    positions: Dict[str, PartSpec]          # named position encodings that mixers refer to
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_position: int

    def validate(self) -> None:
        seen = set()
        for entry in self.schedule:
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule names layer {entry.layer}, the model has {len(self.layers)}")
            seen.add(entry.cache)
        if seen and seen != set(range(len(seen))):
            raise ValueError(f"cache ids of the schedule must be 0..{len(seen) - 1}, got {sorted(seen)}")


class ModelConfig:
    """Base of the typed configurations. A subclass is a dataclass whose fields are the keys of
    the architecture's ``config.json`` and which implements ``from_json`` and ``model_spec``."""

    architecture: str = ""

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_json(self) -> Dict[str, Any]:
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError

    def eos_token_ids(self) -> List[int]:
        return []
