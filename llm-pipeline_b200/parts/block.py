"""Arrangements of a mixer, a feed-forward and their norms around the residual stream.

``pre_norm_residual`` is the decoder layer of
src/llm_pipeline/models/qwen3/custom_builder.py:222-255: ``x += mixer(norm1(x))`` then
``x += feed_forward(norm2(x))``. The sums are not taken here: each part's output is left pending
on the stream and the next norm kernel adds it into the float32 residual."""

from __future__ import annotations

from .base import Block, LayerCache, ResidualStream
from .registry import register_block


@register_block("pre_norm_residual")
class PreNormResidualBlock(Block):
    NORMS = ("mixer", "feed_forward")

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        h = self._norm(self.mixer_norm, self.mixer, stream, ctx)
        out, bias = getattr(self.mixer, "forward_deferred", self.mixer.forward)(h, ctx, cache)
        stream.add(out, bias)
        h = self._norm(self.feed_forward_norm, self.feed_forward, stream, ctx)
        out, bias = getattr(self.feed_forward, "forward_deferred", self.feed_forward.forward)(h, ctx)
        stream.add(out, bias)

    @staticmethod
    def _norm(norm, consumer, stream: ResidualStream, ctx):
        """The norm's rows for ``consumer``: with their factors still to be applied where the norm can leave them so
        and the consumer takes them so."""
        deferred = getattr(norm, "add_norm_deferred", None)
        if deferred is not None and getattr(consumer, "takes_scaled_rows", False):
            return deferred(stream, ctx)
        return norm.add_norm(stream, ctx)
