"""A model assembled from parts according to a ``ModelSpec``.

The same class serves every architecture: the configuration decides which parts each layer has
and in which order layers run (src/llm_pipeline/models/qwen3/custom_builder.py:291-375 for the
Qwen3 order: embedding, the decoder layers, final norm; :378-421 the output head)."""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.spec import PagesSpec, StateSpec
from ..config.base import ModelSpec, PartSpec
from ..ops.linear import begin_step
from ..ops.timing import nvtx_range
from ..parts import LayerCache, ResidualStream, lookup
from ..weights.source import (ParamSpec, TiedWeightError, WeightSource, check_names_and_shapes,
                              stored_dtype_policy)


def _make(family: str, spec: PartSpec):
    return lookup(family, spec.kind)(spec.prefix, **spec.args)


class Model:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = _make("embedding", spec.embedding)
        self.positions = {name: _make("position", p) for name, p in spec.positions.items()}
        self.position_streams = max([int(getattr(p, "streams", 1)) for p in self.positions.values()] or [1])
        self.blocks = []
        for layer in spec.layers:
            block_cls = lookup("block", layer.block)
            self.blocks.append(block_cls(_make("mixer", layer.mixer), _make("feed_forward", layer.feed_forward),
                                         norms={name: _make("norm", norm) for name, norm in layer.named_norms().items()}))
        self.final_norm = _make("norm", spec.final_norm)
        self.head = _make("head", spec.head)
        self.schedule = list(spec.schedule)
        # Which execution owns (writes) each cache id: the first that names it.
        self._owner: Dict[int, int] = {}
        for i, entry in enumerate(self.schedule):
            self._owner.setdefault(entry.cache, i)
        # one mixer of every group whose members answer ``graph_key`` alike (36 equal attention layers: one question)
        self._key_mixers = list({block.mixer.graph_key_group(): block.mixer
                                 for block in (self.blocks[e.layer] for e in self.schedule)}.values())
        self.device: Optional[torch.device] = None
        self.dtype: Optional[torch.dtype] = None

    # -- structure -------------------------------------------------------------------------
    def parts(self):
        yield self.embedding
        yield from self.positions.values()
        for block in self.blocks:
            yield from block.parts()
        yield self.final_norm
        yield self.head

    def expected_params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for part in self.parts():
            for name, spec in part.param_specs().items():
                if name in out and out[name].shape != spec.shape:
                    raise ValueError(f"two parts expect {name} with different shapes")
                out.setdefault(name, spec)
        return out

    def graph_key(self, shape) -> tuple:
        """What the launches of a step of single tokens depend on beyond the number of requests, as the mixers say
        (``Mixer.graph_key``): part of the key of a captured decode step."""
        return tuple(mixer.graph_key(shape) for mixer in self._key_mixers)

    def captured_context_limit(self) -> Optional[int]:
        """The longest context every mixer takes in a captured step (None: any)."""
        limits = [m.captured_context_limit() for m in self._key_mixers]
        limits = [n for n in limits if n is not None]
        return min(limits) if limits else None

    def cache_specs(self) -> List[Tuple[Optional[PagesSpec], Optional[StateSpec]]]:
        """Per cache id, what the layer that owns it asks of the cache manager."""
        count = max((e.cache for e in self.schedule), default=-1) + 1
        specs: List[Tuple[Optional[PagesSpec], Optional[StateSpec]]] = [(None, None)] * count
        for cache_id, index in self._owner.items():
            mixer = self.blocks[self.schedule[index].layer].mixer
            specs[cache_id] = (mixer.cache_spec(), mixer.state_spec())
        return specs

    # -- weights ---------------------------------------------------------------------------
    def load(self, source: WeightSource, device: torch.device, dtype: torch.dtype) -> "Model":
        """Check all names and shapes, then move the tensors to the device part by part."""
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        expected = self.expected_params()
        check_names_and_shapes(expected, source)
        have = set(source.names())
        for part in self.parts():
            for name, original in part.copies().items():
                if name in have and not torch.equal(source.get(name), source.get(original)):
                    raise TiedWeightError(name, original)
        self.device, self.dtype = torch.device(device), dtype
        # A tensor two parts read (the table of a tied head) is moved to the device once.
        tied_to = self.spec.head.args.get("tied_to")
        tied = {f"{tied_to}.weight"} if tied_to else set()
        shared: Dict[tuple, torch.Tensor] = {}

        def get(name: str, role: str) -> torch.Tensor:
            key = (name, role)
            if key in shared:
                return shared[key]
            stored = source.get(name)
            keep = stored_dtype_policy(role, stored.dtype, dtype)
            tensor = stored.to(device=self.device, dtype=keep)
            if name in tied:
                shared[key] = tensor
            return tensor

        for part in self.parts():
            part.load(get)
        shared.clear()
        return self

    # -- one step --------------------------------------------------------------------------
    def forward(self, ctx, caches) -> ResidualStream:
        """Run every scheduled layer on the step's tokens. ``caches.view(cache_id, writes)`` gives
        the ``LayerCache`` of an execution."""
        stream = self.begin(ctx)
        self.run_layers(ctx, caches, stream, 0, len(self.schedule))
        return stream

    def begin(self, ctx) -> ResidualStream:
        """What comes before the first layer: the position tables of the step and the embedded tokens."""
        begin_step()
        with nvtx_range("positions and embedding"):
            ctx.position_tables = {name: part.tables(ctx) for name, part in self.positions.items()}
            return ResidualStream(self.embedding.forward(ctx))

    def run_layers(self, ctx, caches, stream: ResidualStream, first: int, end: int) -> None:
        """The scheduled executions first .. end - 1 on ``stream``."""
        for index in range(first, end):
            entry = self.schedule[index]
            cache = caches.view(entry.cache, writes=self._owner[entry.cache] == index)
            with nvtx_range(f"layer {entry.layer} (execution {index})"):
                self.blocks[entry.layer].forward(stream, ctx, cache)

    def pieces(self) -> List[Tuple[int, int, bool]]:
        """The schedule as runs (first, end, capturable): consecutive executions whose blocks are all ``graph_safe``
        (their work for a step of fixed shape can be captured in a CUDA graph and replayed) and the runs between
        them, which must run eagerly every step. Empty when what surrounds the layers (embedding, position
        encodings, final norm, head) is not capturable: such a model runs eagerly as a whole."""
        safe = lambda part: bool(getattr(part, "graph_safe", False))   # noqa: E731
        around = [self.embedding, self.final_norm, self.head] + list(self.positions.values())
        if not all(safe(part) for part in around):
            return []
        out: List[Tuple[int, int, bool]] = []
        for index, entry in enumerate(self.schedule):
            ok = all(safe(part) for part in self.blocks[entry.layer].parts())
            if out and out[-1][2] == ok:
                out[-1] = (out[-1][0], index + 1, ok)
            else:
                out.append((index, index + 1, ok))
        return out

    def logits(self, ctx, stream: ResidualStream, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] at the given token rows of the step."""
        with nvtx_range("final norm and head"):
            normed = self.final_norm.add_norm(stream, ctx, rows=rows)
            return self.head.forward(normed, ctx)
