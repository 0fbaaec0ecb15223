"""The host-side decisions about attention work (no GPU): which decode kernel a step takes and how the work list of
the general kernel shares a tile's keys among items, for a GPU of 148 SMs."""

from llm_pipeline_b200.parts.attention import AttentionPolicy
from llm_pipeline_b200.ops import kernels

SMS = 148


def takes_list(contexts, kv_heads=8):
    return kernels.decode_prefers_list(max(contexts), sum(contexts), len(contexts), kv_heads, SMS)


def test_even_batches_keep_blocks_of_their_own():
    for contexts in ([2048], [2048] * 8, [16384] * 8, [2048] * 16, [2048] * 32, [8192] * 8 + [100], [300, 200, 250]):
        assert not takes_list(contexts), contexts


def test_uneven_or_many_requests_take_the_list_kernel():
    for contexts in ([131072], [32768, 600], [16384] + [512] * 7, [2048] * 64, [65536, 100, 100, 100],
                     [8000, 100, 3000, 700, 64, 2000, 3000, 5000, 400, 400, 1200, 2048, 2048, 90, 10000, 256]):
        assert takes_list(contexts), contexts


def plan(starts, q_lens, max_segments=8, kv_heads=8, tokens_per_tile=32, first=0):
    return AttentionPolicy.plan_items(starts, q_lens, tokens_per_tile, first, max_segments, kv_heads, SMS)


def items_of(plan_):
    req, tok0, seg, slot, places = plan_
    return list(zip(req, tok0, [s & 255 for s in seg], [s >> 8 for s in seg], slot)), places


def test_whole_tiles_when_blocks_fill_the_sms():
    # a 2,048-token prompt: 64 tiles x 8 heads = 512 blocks
    items, places = items_of(plan([0], [2048]))
    assert places == 0 and len(items) == 64 and all(n == 1 and k == 0 for _, _, k, n, _ in items)
    # sorted by the keys a tile sees
    assert [t for _, t, _, _, _ in items] == list(range(0, 2048, 32))


def test_few_tokens_over_many_keys_share_their_tiles():
    # 512 new tokens over 32,768 keys: 16 tiles x 8 heads = 128 blocks -> 4 items a tile
    items, places = items_of(plan([32768], [512]))
    assert places == 64 and len(items) == 64
    seen = {}
    for at, (r, t, k, n, slot) in enumerate(items):
        assert n == 4 and r == 0
        seen.setdefault(t, []).append((at, k, slot))
    for t, group in seen.items():
        # the items of a tile follow one another, numbered 0.., and share the tile's first place
        assert [k for _, k, _ in group] == [0, 1, 2, 3]
        assert [a for a, _, _ in group] == list(range(group[0][0], group[0][0] + 4))
        assert len({s for _, _, s in group}) == 1 and group[0][2] == group[0][0]
    assert sorted({s for g in seen.values() for _, _, s in g}) == list(range(0, 64, 4))


def test_items_keep_a_minimum_of_keys_and_kernels_without_sharing_get_whole_tiles():
    # 4,096 keys are 33 key tiles: at most 2 items of 16 key tiles
    items, places = items_of(plan([4096], [64]))
    assert places == 4 and all(n == 2 for _, _, _, n, _ in items)
    # short contexts: whole tiles
    items, places = items_of(plan([700], [64]))
    assert places == 0 and all(n == 1 for _, _, _, n, _ in items)
    # a kernel that takes whole tiles only
    items, places = items_of(plan([32768], [512], max_segments=1))
    assert places == 0 and len(items) == 16


def test_requests_before_the_first_are_left_out_and_mixed_lengths_split_by_their_own_keys():
    items, places = items_of(plan([40000, 100, 20000], [1, 40, 33], first=1))
    assert {r for r, *_ in items} == {1, 2}
    by_request = {}
    for r, t, k, n, _ in items:
        by_request.setdefault((r, t), n)
    assert by_request[(1, 0)] == 1 and by_request[(1, 32)] == 1        # 140 keys: whole
    assert by_request[(2, 0)] == 8 and by_request[(2, 32)] == 8        # 20,033 keys: shared
    assert places == 16


def test_decode_graph_shape_at_the_kernels_limit():
    """The block-table width of a decode graph is rounded up to 32 pages; the context bound its kernels are sized for
    never passes what a request may hold, and a bound beyond the decode kernels' limit means: no graph."""
    from llm_pipeline_b200.engine.runner import ModelRunner
    from llm_pipeline_b200.ops import kernels
    limit = kernels.DECODE_MAX_KEYS

    def shape(longest, page, most):
        return ModelRunner.decode_graph_shape(longest, page, most, limit)

    assert shape(2049, 16, 4096) == (160, 2560)                       # 129 pages -> 160; 160 * 16 keys
    assert shape(4000, 16, 4096) == (256, 4096)
    assert shape(4090, 16, 4090) == (256, 4096)                       # the limit of the request, rounded up to a range
    # a request of legal length whose width bucket alone reaches past the limit: clamped, the graph stays
    assert shape(limit - 5, 48, limit) == (2752, limit)
    # a cache made for longer requests than the decode kernels take: eager steps, which refuse only what really is too long
    assert shape(limit - 5, 48, 2 * limit) == (2752, None)
    assert shape(1000, 16, 2 * limit) == (64, 1024)
