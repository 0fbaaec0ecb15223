"""The scheduler's decisions, with the cache manager keeping books only and a stand-in for the
step function that reserves, commits and hands back scripted tokens."""

import pytest

from llm_pipeline_b200.cache import CacheManager, KVPagesSpec
from llm_pipeline_b200.engine.scheduler import Request, Scheduler
from llm_pipeline_b200.sampling import SamplingConfig


def make(num_pages=64, page_size=4, max_seqs=4, budget=16, chunk=None, max_len=256):
    cache = CacheManager([(KVPagesSpec(1, 16), None)], page_size=page_size, num_pages=num_pages, max_requests=8,
                         max_request_tokens=max_len, device=None)
    return cache, Scheduler(cache, max_seqs, budget, max_len, chunk)


def request(rid, prompt_len, max_tokens=4, eos=()):
    return Request(rid, list(range(1, prompt_len + 1)), SamplingConfig(), max_tokens, set(eos))


def run_step(cache, sched, token=lambda req: 100 + len(req.output)):
    """What the engine does around a plan: admit, reserve, commit, sample."""
    plan = sched.schedule()
    for e in plan.entries:
        if e.request.req_id not in cache:
            cache.admit(e.request.req_id)
        assert e.start == cache.length(e.request.req_id)
        assert cache.reserve(e.request.req_id, e.start + e.count), "the plan must fit the pages"
        cache.commit(e.request.req_id, e.start + e.count)
    sampled = {e.request.req_id: token(e.request) for e in plan.entries if e.samples}
    finished = sched.finish_step(plan, sampled)
    cache.check()
    return plan, finished


def test_prompt_is_cut_under_the_token_budget_and_then_decodes():
    cache, sched = make(budget=16)
    sched.add(request("a", 40, max_tokens=3))
    sizes, samples = [], []
    while sched.has_unfinished():
        plan, _ = run_step(cache, sched)
        sizes.append([e.count for e in plan.entries])
        samples.append([e.samples for e in plan.entries])
    assert sizes == [[16], [16], [8], [1], [1]]
    assert samples == [[False], [False], [True], [True], [True]]
    assert cache.num_live == 0 and cache.groups[0].pool.num_free == 64


def test_decodes_go_first_and_prompts_fill_the_rest():
    cache, sched = make(budget=12, chunk=8)
    sched.add(request("a", 5, max_tokens=8))
    run_step(cache, sched)                      # a: whole prompt, first token
    sched.add(request("b", 30, max_tokens=2))
    sched.add(request("c", 6, max_tokens=2))
    plan, _ = run_step(cache, sched)
    assert [(e.request.req_id, e.count, e.samples) for e in plan.entries] == [("a", 1, True), ("b", 8, False), ("c", 3, False)]
    plan, _ = run_step(cache, sched)            # a decodes; b (admitted first) continues; c gets what is left
    assert [(e.request.req_id, e.count) for e in plan.entries] == [("a", 1), ("b", 8), ("c", 3)]
    assert plan.num_tokens <= 12


def test_admission_is_limited_by_sequences_and_keeps_arrival_order():
    cache, sched = make(max_seqs=2, budget=64)
    for rid, n in (("a", 4), ("b", 4), ("c", 4)):
        sched.add(request(rid, n, max_tokens=2))
    plan, _ = run_step(cache, sched)
    assert [e.request.req_id for e in plan.entries] == ["a", "b"] and [r.req_id for r in sched.waiting] == ["c"]
    plan, finished = run_step(cache, sched)     # a and b finish (2 tokens), c still waits in this step
    assert sorted(r.req_id for r in finished) == ["a", "b"]
    plan, _ = run_step(cache, sched)
    assert [e.request.req_id for e in plan.entries] == ["c"]


def test_finish_on_eos_length_and_model_len():
    cache, sched = make(max_len=12)
    sched.add(request("eos", 3, max_tokens=10, eos={101}))
    sched.add(request("len", 3, max_tokens=2))
    sched.add(request("ctx", 9, max_tokens=50))
    reasons = {}
    while sched.has_unfinished():
        _, finished = run_step(cache, sched)
        reasons.update({r.req_id: (r.finish_reason, len(r.output)) for r in finished})
    assert reasons == {"eos": ("stop", 2), "len": ("length", 2), "ctx": ("length", 3)}
    with pytest.raises(ValueError, match="no room"):
        sched.add(request("big", 12))
    with pytest.raises(ValueError, match="empty"):
        sched.add(request("none", 0))


def test_waiting_request_is_not_admitted_without_pages_and_nobody_overtakes():
    cache, sched = make(num_pages=6, page_size=4, budget=64)       # 24 tokens in all
    sched.add(request("a", 14, max_tokens=6))
    sched.add(request("b", 12, max_tokens=2))
    sched.add(request("c", 2, max_tokens=2))
    plan, _ = run_step(cache, sched)
    assert [e.request.req_id for e in plan.entries] == ["a"]       # b needs 3 pages, 2 are free; c stays behind b
    assert [r.req_id for r in sched.waiting] == ["b", "c"] and not plan.preempted


def test_running_out_of_pages_preempts_the_newest_and_recomputes_it():
    cache, sched = make(num_pages=6, page_size=4, budget=64)
    sched.add(request("a", 11, max_tokens=12))
    sched.add(request("b", 9, max_tokens=12))
    run_step(cache, sched)                                          # a: 3 pages, b: 3 pages -> pool is full
    outputs_before = None
    preempted_at = None
    for step in range(40):
        plan, _ = run_step(cache, sched)
        if plan.preempted and preempted_at is None:
            preempted_at = step
            assert [r.req_id for r in plan.preempted] == ["b"]      # the request admitted last
            assert sched.waiting[0].req_id == "b" and sched.waiting[0].computed == 0
            assert "b" not in cache
            assert [e.request.req_id for e in plan.entries] == ["a"]
            outputs_before = list(sched.waiting[0].output)
        if not sched.has_unfinished():
            break
    assert preempted_at is not None and sched.num_preemptions >= 1
    assert not sched.has_unfinished() and cache.num_live == 0
    assert cache.groups[0].pool.num_free == 6
    assert outputs_before is not None


def test_preempted_request_is_recomputed_from_prompt_plus_output():
    cache, sched = make(num_pages=5, page_size=4, budget=64)
    a, b = request("a", 8, max_tokens=9), request("b", 7, max_tokens=9)
    sched.add(a)
    sched.add(b)
    done = {}
    portions = []
    for _ in range(60):
        plan, finished = run_step(cache, sched)
        portions += [(e.request.req_id, e.start, e.count) for e in plan.entries if e.request is b]
        done.update({r.req_id: r for r in finished})
        if not sched.has_unfinished():
            break
    assert set(done) == {"a", "b"} and b.preemptions >= 1
    restarts = [p for p in portions if p[1] == 0]
    assert len(restarts) == 1 + b.preemptions
    assert restarts[1][2] > 7                    # the recomputation covers the prompt and the generated tokens
    assert done["b"].output == [100 + i for i in range(9)]       # every token sampled once, in order


def test_a_single_request_that_cannot_fit_is_finished_not_looped():
    cache, sched = make(num_pages=2, page_size=4, budget=64)
    sched.add(request("a", 6, max_tokens=50))
    reasons = []
    for _ in range(10):
        plan, finished = run_step(cache, sched)
        reasons += [r.finish_reason for r in finished] + [r.finish_reason for r in plan.aborted]
        if not sched.has_unfinished():
            break
    assert reasons == ["out_of_pages"] and cache.num_live == 0
    sched.add(request("b", 20, max_tokens=2))                     # cannot even start
    plan, _ = run_step(cache, sched)
    assert [r.finish_reason for r in plan.aborted] == ["out_of_pages"] and not sched.has_unfinished()


def test_abort_frees_pages():
    cache, sched = make()
    sched.add(request("a", 9))
    run_step(cache, sched)
    assert sched.abort("a").finish_reason == "abort" and cache.num_live == 0 and not sched.has_unfinished()


def test_position_ids_of_a_portion_go_on_after_the_prompts_largest_id():
    """A request may bring position ids in several streams for its prompt; portions take their slices, and generated
    tokens (also when a preempted request is recomputed from prompt plus output) count on from the largest id."""
    r = Request("a", [5, 6, 7, 8], SamplingConfig(), 8, position_ids=[[0, 0, 1, 1], [0, 1, 0, 9]])
    assert r.positions_of(0, 4) == [[0, 0, 1, 1], [0, 1, 0, 9]]
    assert r.positions_of(1, 2) == [[0, 1], [1, 0]]
    r.output = [3, 3, 3]
    assert r.positions_of(4, 1) == [[10], [10]]
    assert r.positions_of(6, 1) == [[12], [12]]
    assert r.positions_of(2, 4) == [[1, 1, 10, 11], [0, 9, 10, 11]]
    assert Request("b", [1, 2], SamplingConfig(), 4).positions_of(0, 2) is None


def test_tokens_that_reach_the_host_a_step_late():
    """The engine may plan a step before it has read what the step before sampled: a token given as None counts
    towards the lengths and is planned as the request's next input; ``late_token`` brings its value. A request that is
    full leaves as "draining" and is finished when its last token arrives; an end-of-sequence token that arrives late
    ends its request there and then, and what was sampled after it is dropped."""
    from llm_pipeline_b200.engine.scheduler import PENDING
    cache, sched = make(num_pages=16, budget=64, max_len=64)

    def run(cache, plan):
        for e in plan.entries:
            if e.request.req_id not in cache:
                cache.admit(e.request.req_id)
            assert cache.reserve(e.request.req_id, e.start + e.count)
            cache.commit(e.request.req_id, e.start + e.count)

    a = Request("a", [1, 2, 3], SamplingConfig(), 3, eos_token_ids={9})
    b = Request("b", [4, 5], SamplingConfig(), 8, eos_token_ids={9})
    sched.add(a)
    sched.add(b)
    plan = sched.schedule()
    assert [(e.request.req_id, e.count, e.samples) for e in plan.entries] == [("a", 3, True), ("b", 2, True)]
    run(cache, plan)
    assert sched.finish_step(plan, {"a": None, "b": None}) == []
    assert a.in_flight == 1 and a.output == [] and a.tokens == [1, 2, 3, PENDING] and a.num_pending == 1
    plan2 = sched.schedule()                                   # planned without knowing the tokens
    assert [(e.request.req_id, e.token_ids, e.samples) for e in plan2.entries] == [("a", [PENDING], True), ("b", [PENDING], True)]
    run(cache, plan2)
    assert sched.finish_step(plan2, {"a": None, "b": None}) == []
    assert not sched.late_token(a, 7)
    assert sched.late_token(b, 9)                              # b's first token ends it
    assert b.status == "finished" and b.finish_reason == "stop" and b.output == [9] and b.in_flight == 1 and "b" not in cache
    assert a.output == [7] and a.in_flight == 1 and a.status == "running"
    plan3 = sched.schedule()                                   # a's third and last token
    assert [e.request.req_id for e in plan3.entries] == ["a"]
    run(cache, plan3)
    assert sched.finish_step(plan3, {"a": None}) == [] and a.status == "draining" and "a" not in cache
    assert not sched.has_unfinished()
    assert not sched.late_token(b, 5) and b.output == [9] and b.in_flight == 0        # sampled in vain: dropped
    assert not sched.late_token(a, 8) and a.status == "draining"
    assert sched.late_token(a, 6) and a.status == "finished" and a.finish_reason == "length" and a.output == [7, 8, 6]
    cache.check()


def test_a_portion_of_a_requests_tokens_without_putting_them_all_together():
    import random
    from llm_pipeline_b200.engine.scheduler import PENDING
    rng = random.Random(0)
    for _ in range(500):
        r = Request("a", [rng.randrange(100) for _ in range(rng.randrange(1, 8))], SamplingConfig(), 10)
        r.output = [rng.randrange(100) for _ in range(rng.randrange(0, 6))]
        r.in_flight = rng.randrange(0, 3)
        whole = r.tokens
        assert whole[len(whole) - r.in_flight:] == [PENDING] * r.in_flight
        start = rng.randrange(0, len(whole) + 1)
        count = rng.randrange(0, len(whole) - start + 2)
        assert r.token_slice(start, count) == whole[start:start + count]
