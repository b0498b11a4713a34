"""The scheduler's decisions, on the host with a cache manager that has no device: admission,
the token budget and portions, decoding, finishing and freeing, and what happens when pages
run out (preemption of the request admitted last, recomputation, refusal at submission)."""
import random

import pytest

from spyinfer_b200.cache import CacheManager
from spyinfer_b200.config import EngineConfig, PagedCacheNeed
from spyinfer_b200.engine.scheduler import RequestTooLarge, Scheduler
from spyinfer_b200.engine.sequence import Sequence, SequenceStatus
from spyinfer_b200.sampling import SamplingParams


def make(num_pages=16, page_size=4, budget=32, max_num_seqs=4, max_model_len=64, chunk_size=None):
    cfg = EngineConfig(max_num_batched_tokens=budget, max_num_seqs=max_num_seqs, max_model_len=max_model_len, chunk_size=chunk_size,
                       kvcache_block_size=page_size, num_kvcache_blocks=num_pages)
    cache = CacheManager([PagedCacheNeed(1, 16, None)], page_size, num_pages, max_num_seqs, max_model_len, device=None)
    return Scheduler(cfg, cache), cache


def seq(i, n, max_new=8):
    return Sequence(i, list(range(n)), n, SamplingParams(max_new_tokens=max_new))


def run_step(sched, cache, portions, next_token=7):
    """What the engine does with a step's portions: runs them, commits, appends samples, finishes."""
    finished = []
    for p in portions:
        assert p.start == p.seq.num_computed == cache.length(p.seq.id)
        cache.commit(p.seq.id, p.start + p.num_tokens)
        p.seq.num_computed = p.start + p.num_tokens
        assert p.samples == (p.seq.num_computed == len(p.seq))
        if p.samples:
            p.seq.tokens.append(next_token)
            if p.seq.num_generated >= p.seq.sampling.max_new_tokens:
                sched.finish(p.seq, "max_new_tokens")
                finished.append(p.seq.id)
    cache.check_invariants()
    return finished


def test_admission_is_first_come_first_served_under_the_budget():
    sched, cache = make(budget=20)
    a, b, c = seq(0, 12), seq(1, 12), seq(2, 3)
    for s in (a, b, c):
        sched.add_sequence(s)
    p = sched.schedule()
    assert [(x.seq.id, x.start, x.num_tokens, x.samples) for x in p] == [(0, 0, 12, True), (1, 0, 8, False)]
    assert c.status == SequenceStatus.WAITING            # the budget was spent before c's turn
    run_step(sched, cache, p)
    p = sched.schedule()
    # decoding first (a), then the rest of b's prompt, then c is admitted
    assert [(x.seq.id, x.start, x.num_tokens, x.samples) for x in p] == [(0, 12, 1, True), (1, 8, 4, True), (2, 0, 3, True)]


def test_prompt_is_cut_into_portions_by_the_budget():
    sched, cache = make(num_pages=32, budget=5, max_model_len=128)
    a = seq(0, 17, max_new=2)
    sched.add_sequence(a)
    sizes = []
    while sched.has_unfinished():
        p = sched.schedule()
        sizes.append([(x.start, x.num_tokens) for x in p])
        run_step(sched, cache, p)
    assert sizes == [[(0, 5)], [(5, 5)], [(10, 5)], [(15, 2)], [(17, 1)]]
    assert a.status == SequenceStatus.FINISHED and a.finish_reason == "max_new_tokens"
    assert cache.num_free_pages() == 32 and cache.num_free_slots() == 4


def test_chunk_size_caps_each_requests_portion_beside_the_budget():
    """Two prompts under a budget of 16 and a chunk size of 6: each gets at most 6 tokens a step, both
    run in the same step, and a decoding request still gets its one token first."""
    sched, cache = make(num_pages=32, budget=16, max_model_len=128, chunk_size=6)
    a, b = seq(0, 14, max_new=3), seq(1, 9, max_new=2)
    sched.add_sequence(a)
    sched.add_sequence(b)
    seen = []
    while sched.has_unfinished():
        p = sched.schedule()
        seen.append([(x.seq.id, x.start, x.num_tokens) for x in p])
        run_step(sched, cache, p)
    assert seen[:3] == [[(0, 0, 6), (1, 0, 6)], [(0, 6, 6), (1, 6, 3)], [(1, 9, 1), (0, 12, 2)]]
    assert all(n <= 6 for step in seen for _, _, n in step)
    assert cache.num_free_pages() == 32
    with pytest.raises(ValueError):
        make(chunk_size=0)


def test_max_num_seqs_limits_live_requests():
    sched, cache = make(max_num_seqs=2, budget=64)
    for i in range(3):
        sched.add_sequence(seq(i, 2, max_new=1))
    p = sched.schedule()
    assert [x.seq.id for x in p] == [0, 1]
    run_step(sched, cache, p)                            # both finish after one token
    assert [x.seq.id for x in sched.schedule()] == [2]


def test_admission_waits_for_pages_and_the_head_blocks_those_behind():
    sched, cache = make(num_pages=4, budget=64)          # 16 tokens of cache
    sched.add_sequence(seq(0, 10, max_new=2))
    sched.add_sequence(seq(1, 9, max_new=2))             # needs 3 pages; 1 is free
    sched.add_sequence(seq(2, 2, max_new=2))             # would fit, but must not overtake
    p = sched.schedule()
    assert [x.seq.id for x in p] == [0]
    run_step(sched, cache, p)
    assert [x.seq.id for x in sched.schedule()] == [0]


def test_pages_run_out_while_decoding_preempts_the_newest():
    sched, cache = make(num_pages=4, page_size=4, budget=64)
    a, b = seq(0, 8, max_new=8), seq(1, 8, max_new=8)
    sched.add_sequence(a)
    sched.add_sequence(b)
    run_step(sched, cache, sched.schedule())             # both prompts: 2 pages each, pool full, lengths 9 after sampling
    p = sched.schedule()                                 # position 8 needs a third page for each
    assert [x.seq.id for x in p] == [0]
    assert b.status == SequenceStatus.WAITING and b.num_computed == 0 and b.num_preemptions == 1 and len(b) == 9
    assert sched.waiting[0] is b and not cache.has_request(1)
    cache.check_invariants()
    # a runs on; b comes back when pages are free and is recomputed from all its tokens so far
    steps = 0
    while sched.has_unfinished():
        p = sched.schedule()
        assert p, "the scheduler must always make progress"
        for x in p:
            if x.seq is b and x.start == 0:
                assert x.num_tokens == len(b)            # prompt and generated tokens are run again
        run_step(sched, cache, p)
        steps += 1
        assert steps < 100
    assert a.num_generated == 8 and b.num_generated == 8
    assert cache.num_free_pages() == 4


def test_a_request_that_can_never_fit_is_refused_at_submission():
    sched, cache = make(num_pages=4, page_size=4, max_model_len=64)
    with pytest.raises(RequestTooLarge):
        sched.check_fits(seq(0, 10), max_new_tokens=8)   # 18 tokens need 5 pages
    sched.check_fits(seq(0, 10), max_new_tokens=6)       # 16 tokens fit exactly
    with pytest.raises(RequestTooLarge):
        sched.check_fits(seq(0, 64), max_new_tokens=1)   # no room to generate


def test_tight_pool_and_small_budget_always_make_progress():
    sched, cache = make(num_pages=4, page_size=4, budget=6, max_model_len=64)
    a, b = seq(0, 12, max_new=2), seq(1, 12, max_new=2)
    sched.add_sequence(a)
    sched.add_sequence(b)
    steps = 0
    while sched.has_unfinished():
        p = sched.schedule()
        assert p
        run_step(sched, cache, p)
        steps += 1
        assert steps < 100
    assert a.num_generated == 2 and b.num_generated == 2 and cache.num_free_pages() == 4


@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_finish_with_everything_given_back(seed):
    rng = random.Random(seed)
    chunk = rng.choice([None, None, 2, 5])
    sched, cache = make(num_pages=12, page_size=4, budget=rng.choice([3, 8, 32]), max_num_seqs=3, max_model_len=40, chunk_size=chunk)
    seqs = []
    for i in range(12):
        s = seq(i, rng.randint(1, 20), max_new=rng.randint(1, 12))
        sched.check_fits(s, s.sampling.max_new_tokens)
        seqs.append(s)
    pending = list(seqs)
    steps = 0
    while sched.has_unfinished() or pending:
        while pending and rng.random() < 0.5:
            sched.add_sequence(pending.pop(0))
        p = sched.schedule()
        assert sum(x.num_tokens for x in p) <= sched.config.max_num_batched_tokens
        assert chunk is None or all(x.num_tokens <= chunk for x in p)
        assert len({x.seq.id for x in p}) == len(p) and len(sched.running) <= 3
        run_step(sched, cache, p)
        steps += 1
        assert steps < 2000
    assert all(s.status == SequenceStatus.FINISHED and s.num_generated == s.sampling.max_new_tokens for s in seqs)
    assert cache.num_free_pages() == 12 and cache.num_free_slots() == 3
