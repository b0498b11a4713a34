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


def run_step(sched, cache, portions, next_token=7, cap_at_pool=True):
    """What the engine does with a step's portions: runs them, commits, appends samples, finishes
    (by count, by ``max_model_len``, and, as ``LLMEngine`` does, at the last token that the pool
    could hold for a request alone; ``cap_at_pool=False`` leaves that to the scheduler)."""
    finished = []
    for p in portions:
        assert p.start == p.seq.num_computed == cache.length(p.seq.id)
        cache.commit(p.seq.id, p.start + p.num_tokens)
        p.seq.num_computed = p.start + p.num_tokens
        assert p.samples == (p.seq.num_computed == len(p.seq))
        if p.samples:
            p.seq.tokens.append(next_token)
            limit = p.seq.sampling.max_new_tokens
            if limit is not None and p.seq.num_generated >= limit:
                sched.finish(p.seq, "max_new_tokens")
            elif len(p.seq) >= sched.config.max_model_len:
                sched.finish(p.seq, "max_model_len")
            elif cap_at_pool and len(p.seq) > sched.most_tokens_alone():
                sched.finish(p.seq, "out_of_pages")
            if p.seq.status == SequenceStatus.FINISHED:
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


@pytest.mark.parametrize("cap_at_pool", [True, False])
def test_a_lone_request_without_a_token_limit_ends_where_the_pool_ends(cap_at_pool):
    """4 pages of 4 tokens, ``max_model_len`` 64, no ``max_new_tokens``: the request may grow to 64
    tokens, the pool holds 16.  It is admitted (it may meet its end-of-sequence token early), runs to
    the pool's last token and ends there with the reason "out_of_pages": through the engine's own
    check, or, without it, by the scheduler, which never preempts the only running request."""
    sched, cache = make(num_pages=4, page_size=4, budget=64, max_model_len=64)
    a = seq(0, 10, max_new=None)
    sched.check_fits(a, 1)
    sched.add_sequence(a)
    steps = 0
    while sched.has_unfinished():
        p = sched.schedule()
        run_step(sched, cache, p, cap_at_pool=cap_at_pool)
        steps += 1
        assert steps <= 8, "one prompt step and six or seven decode steps, then the end"
    assert a.status == SequenceStatus.FINISHED and a.finish_reason == "out_of_pages"
    assert len(a) == 17 and a.num_preemptions == 0 and sched.num_preemptions == 0
    assert (sched.ended_without_token == [a]) == (not cap_at_pool)
    assert cache.num_free_pages() == 4 and cache.num_free_slots() == 4


def test_an_unlimited_request_gives_way_then_ends_and_the_preempted_one_comes_back():
    """Two requests without a token limit in a pool that holds neither to ``max_model_len``: the newer
    one is preempted once for the older, the older ends at the pool's end, the newer is recomputed,
    runs on alone and ends there too.  No request is preempted in favour of nobody."""
    sched, cache = make(num_pages=4, page_size=4, budget=64, max_model_len=64)
    a, b = seq(0, 6, max_new=None), seq(1, 6, max_new=None)
    sched.add_sequence(a)
    sched.add_sequence(b)
    steps = 0
    while sched.has_unfinished():
        run_step(sched, cache, sched.schedule(), cap_at_pool=False)
        steps += 1
        assert steps < 40
    assert a.finish_reason == b.finish_reason == "out_of_pages" and len(a) == len(b) == 17
    assert a.num_preemptions == 0 and b.num_preemptions == 1
    assert cache.num_free_pages() == 4 and cache.num_free_slots() == 4


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
        s = seq(i, rng.randint(1, 20), max_new=rng.choice([None, rng.randint(1, 12), rng.randint(1, 12)]))
        sched.check_fits(s, s.sampling.max_new_tokens or 1)
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
    for s in seqs:
        assert s.status == SequenceStatus.FINISHED
        if s.sampling.max_new_tokens is not None:
            assert s.num_generated == s.sampling.max_new_tokens and s.finish_reason == "max_new_tokens"
        else:
            assert len(s) == 40 and s.finish_reason == "max_model_len"     # the pool holds 48 tokens, max_model_len is 40
    assert cache.num_free_pages() == 12 and cache.num_free_slots() == 3


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_in_a_pool_smaller_than_max_model_len(seed):
    """As above, but the pool (24 tokens) is smaller than ``max_model_len`` (40) and a third of the
    requests have no token limit; half of the runs leave the pool's cap to the scheduler."""
    rng = random.Random(100 + seed)
    sched, cache = make(num_pages=6, page_size=4, budget=rng.choice([3, 8, 32]), max_num_seqs=3, max_model_len=40, chunk_size=rng.choice([None, 5]))
    seqs = []
    for i in range(10):
        s = seq(i, rng.randint(1, 14), max_new=rng.choice([None, rng.randint(1, 8), rng.randint(1, 8)]))
        sched.check_fits(s, s.sampling.max_new_tokens or 1)
        seqs.append(s)
    pending = list(seqs)
    steps = 0
    while sched.has_unfinished() or pending:
        while pending and rng.random() < 0.5:
            sched.add_sequence(pending.pop(0))
        run_step(sched, cache, sched.schedule(), cap_at_pool=seed % 2 == 0)
        steps += 1
        assert steps < 2000
    for s in seqs:
        assert s.status == SequenceStatus.FINISHED
        if s.sampling.max_new_tokens is None:
            assert s.finish_reason == "out_of_pages" and len(s) == 25
        else:
            assert s.finish_reason == "max_new_tokens" and s.num_generated == s.sampling.max_new_tokens
    assert cache.num_free_pages() == 6 and cache.num_free_slots() == 3


def test_padded_sizes_of_small_steps():
    """The sizes a small step is padded to for its CUDA graph: few distinct ones, always room for the step and for the
    request that holds the padding tokens, and no padding where there is no room or nothing to gain."""
    from spyinfer_b200.engine.runner import padded_step_sizes
    assert padded_step_sizes(17, 3, 3, 8, 2048, 384) == (32, 4, 4, 0)
    assert padded_step_sizes(32, 1, 1, 8, 2048, 384) == (32, 1, 1, 0)          # nothing to pad
    assert padded_step_sizes(40, 5, 1, 8, 2048, 384) == (64, 8, 8, 0)          # wanted rows: at least one a request
    assert padded_step_sizes(33, 8, 2, 8, 2048, 384) is None                # the padding tokens would need a ninth request
    assert padded_step_sizes(64, 8, 8, 8, 2048, 384) == (64, 8, 8, 0)
    assert padded_step_sizes(130, 2, 1, 64, 2048, 384) == (192, 4, 4, 0)
    assert padded_step_sizes(385, 1, 1, 64, 2048, 384) is None              # large steps run as they are
    assert padded_step_sizes(100, 1, 0, 64, 2048, 384) is None              # nothing wanted: no logits to return
    assert padded_step_sizes(300, 1, 1, 64, 256, 384) is None               # beyond the staging buffers
    assert padded_step_sizes(100, 4, 4, 64, 2048, 384, head=3) == (128, 8, 8, 4)   # three one-token requests at the head and one of padding
    assert padded_step_sizes(31, 2, 2, 8, 2048, 384, head=1) == (32, 4, 4, 1)
    seen = set()
    for t in range(1, 385):
        for s_ in (1, 2, 3, 5, 9, 17, 33):
            sizes = padded_step_sizes(t, s_, min(s_, t), 64, 2048, 384)
            assert sizes is not None and sizes[0] >= t and sizes[1] >= s_ + (1 if sizes[0] > t else 0) and sizes[2] >= min(s_, t)
            seen.add(sizes)
    assert len(seen) <= 60
