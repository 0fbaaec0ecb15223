"""The residual stream's pending addend (no GPU): a product not yet taken is taken when somebody reads it as a
tensor, and handed over untaken only to a norm that asks for it."""

import pytest
import torch

from llm_pipeline_b200.ops.linear import PendingProduct
from llm_pipeline_b200.parts.base import ResidualStream


class CountedProduct(PendingProduct):
    taken = 0

    def value(self):
        CountedProduct.taken += 1
        return self.x @ self.weight.t()


def make():
    CountedProduct.taken = 0
    x, w = torch.randn(3, 4), torch.randn(5, 4)
    return ResidualStream(torch.zeros(3, 5)), CountedProduct(x, w), x @ w.t()


def test_reading_pending_takes_the_product_once():
    stream, product, want = make()
    stream.add(product)
    assert CountedProduct.taken == 0
    assert torch.equal(stream.pending, want) and torch.equal(stream.pending, want)
    assert CountedProduct.taken == 1
    assert stream.take_pending_product() is None            # it is a tensor now
    stream.pending, stream.pending_bias = None, None
    stream.add(torch.ones(3, 5))                            # the stream is free again
    with pytest.raises(RuntimeError):
        stream.add(torch.ones(3, 5))


def test_a_norm_may_take_the_product_untaken():
    stream, product, _ = make()
    stream.add(product)
    assert stream.take_pending_product() is product and CountedProduct.taken == 0
    assert stream.pending is None
    stream.add(torch.ones(3, 5))                            # nothing pending any more: the next part may add


def test_a_product_with_a_bias_is_not_handed_over():
    stream, product, want = make()
    stream.add(product, torch.ones(5))
    assert stream.take_pending_product() is None and CountedProduct.taken == 0
    assert torch.equal(stream.pending, want)
