"""Interfaces of the parts a model is put together from.

Every part takes its sizes and constants as constructor parameters, declares the tensors it
expects (``param_specs``: full tensor name -> ``ParamSpec``), receives them through ``load`` and
works on the tensors of one step. No part knows which model it is in.

* ``Norm.add_norm(stream, rows=None)``: folds the stream's pending sum into the float32 residual
  and returns the normalised rows in the compute type.
* ``PositionEncoding.tables(ctx)``: per-step tensors derived from the token positions (for the
  rotary kind: float32 cos/sin ``[tokens, rotary_dim / 2]``).
* ``Mixer.forward(x, ctx, cache) -> (out, bias)``: mixes tokens of the same request; ``cache`` is
  the ``LayerCache`` of this execution (pages and/or a state tensor). ``cache_spec()`` and
  ``state_spec()`` tell the cache manager what it needs.
* ``FeedForward.forward(x, ctx) -> (out, bias)``: works on each token alone.
* ``Block.forward(stream, ctx, cache)``: the arrangement of the above around the residual stream.

Optional, for the few rows of a decode step (``ops/linear.py``: a norm between two streaming products folded into
them): a mixer or feed-forward with ``forward_deferred(...)`` may return its last product as a ``PendingProduct``; a
norm with ``add_norm_deferred(stream, ctx)`` may take such a product from the stream and return ``ScaledRows``; a part
that sets ``takes_scaled_rows`` accepts those as its ``x`` (``linear()`` does). A block uses these only where both
sides offer them; parts without them see tensors only.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Hashable, Optional, Tuple

import torch

from ..cache.spec import KVPagesSpec, PagesSpec, StateSpec
from ..ops.linear import PendingProduct
from ..weights.source import ParamSpec

TensorGetter = Callable[[str, str], torch.Tensor]   # (full tensor name, role) -> tensor on the device


@dataclass
class LayerCache:
    """What one execution of a layer may touch: the pages of its cache id (``writes`` is False when
    an earlier execution owns them), the index of their group (for block tables and slot
    mappings in the step context), and the state tensor ``[slots, ...]`` of its cache id."""

    pages: Optional[torch.Tensor] = None
    group: Optional[int] = None
    state: Optional[torch.Tensor] = None
    writes: bool = True


class ResidualStream:
    """The hidden state between parts: a float32 residual ``[tokens, hidden]`` and a pending
    addend in the compute type (with an optional bias vector) that the next norm folds in."""

    def __init__(self, residual: torch.Tensor):
        self.residual = residual
        self._pending = None
        self.pending_bias: Optional[torch.Tensor] = None

    def add(self, delta, bias: Optional[torch.Tensor] = None) -> None:
        """``delta``: a tensor, or a product not yet taken (``ops.linear.PendingProduct``) that the next norm may
        fold into its own work."""
        if self._pending is not None:
            raise RuntimeError("the residual stream already holds a pending addend")
        self._pending, self.pending_bias = delta, bias

    @property
    def pending(self) -> Optional[torch.Tensor]:
        """The pending addend as a tensor (a product not yet taken is taken now)."""
        if isinstance(self._pending, PendingProduct):
            self._pending = self._pending.value()
        return self._pending

    @pending.setter
    def pending(self, delta) -> None:
        self._pending = delta

    def settle(self) -> torch.Tensor:
        """Add what is pending into the residual and return it: the whole state of the stream in one float32 tensor
        (between pieces of a step that are captured apart; the norms fold the addend in on their own otherwise)."""
        pending = self.pending
        if pending is not None:
            self.residual = self.residual + pending.float()
            if self.pending_bias is not None:
                self.residual = self.residual + self.pending_bias.float()
            self._pending, self.pending_bias = None, None
        return self.residual

    def take_pending_product(self) -> Optional[PendingProduct]:
        """The pending addend if it is a product not yet taken and without bias, which is then the caller's to add;
        else None, and nothing changes."""
        if isinstance(self._pending, PendingProduct) and self.pending_bias is None:
            product, self._pending = self._pending, None
            return product
        return None


class Part:
    prefix: str = ""
    # True when the part's work for a step can be captured in a CUDA graph and replayed: fixed launch
    # shapes for fixed step shapes, no host synchronisation, and running the step twice leaves the same
    # state. The built-in parts are; a part that does not say so keeps the whole model on eager steps.
    graph_safe: bool = False

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def copies(self) -> Dict[str, str]:
        """Names of optional tensors of this part that, where a checkpoint holds them, must repeat
        another tensor: {own name: the name it repeats}. The loader compares the two."""
        return {}

    def load(self, get: TensorGetter) -> None:
        pass


class Norm(Part):
    def add_norm(self, stream: ResidualStream, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    # Streams of position ids the encoding reads for every token: ``ctx.position_ids`` is [streams of the model, N].
    # With one stream (the default) that is each token's place in its request; an encoding with more (a place along
    # several axes) gets what the request brought (``StepEntry.positions``), or the place in every stream.
    streams: int = 1

    def tables(self, ctx):
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self) -> Optional[PagesSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def graph_key(self, shape) -> Hashable:
        """For a mixer whose launches for a step of single tokens depend on more than the number of requests: what they
        depend on, as a hashable value (``shape``: ``engine.StepShape``). It becomes part of the key under which the step
        function captures and replays such steps. None: nothing."""
        return None

    def captured_context_limit(self) -> Optional[int]:
        """The longest context (keys a request sees) for which the mixer's kernels can be sized in a captured step of
        single tokens; None: any. Mixers of one ``graph_key_group`` answer alike."""
        return None

    def graph_key_group(self) -> Hashable:
        """Mixers that return equal values here give equal ``graph_key`` for every step; the model then asks one of
        them. The default keeps every mixer apart."""
        return id(self)

    def forward(self, x: torch.Tensor, ctx, cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx) -> torch.Tensor:
        """float32 residual [tokens, hidden] of ctx.token_ids"""
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """float32 logits [rows, vocab]"""
        raise NotImplementedError


class Block:
    """An arrangement of a mixer, a feed-forward and named norms around the residual stream. ``norms`` maps the
    names of ``LayerSpec.named_norms()`` to the built norms; the two of a pre-norm block may also come as the third
    and fourth argument. ``NORMS`` lists the names a block kind needs; building a layer without one of them fails."""

    NORMS: Tuple[str, ...] = ()

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Optional[Norm] = None,
                 feed_forward_norm: Optional[Norm] = None, norms: Optional[Dict[str, Norm]] = None):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms: Dict[str, Norm] = {}
        if mixer_norm is not None:
            self.norms["mixer"] = mixer_norm
        if feed_forward_norm is not None:
            self.norms["feed_forward"] = feed_forward_norm
        self.norms.update(norms or {})
        missing = [name for name in self.NORMS if name not in self.norms]
        if missing:
            raise ValueError(f"a {type(self).__name__} needs the norms {list(self.NORMS)}; the layer lacks {missing}")

    @property
    def mixer_norm(self) -> Optional[Norm]:
        return self.norms.get("mixer")

    @property
    def feed_forward_norm(self) -> Optional[Norm]:
        return self.norms.get("feed_forward")

    def parts(self):
        return tuple(self.norms.values()) + (self.mixer, self.feed_forward)

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        raise NotImplementedError
