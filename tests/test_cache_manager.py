"""The cache manager on the host: pages, block tables, groups, windows, state slots."""
import random

import pytest

from spyinfer_b200.cache import CacheManager, NoFreeSlot, OutOfPages, PagePool
from spyinfer_b200.config import PagedCacheNeed, StateCacheNeed

FULL = PagedCacheNeed(2, 16, None)
WIN = PagedCacheNeed(2, 16, 10)


def manager(needs=(FULL, FULL), page_size=4, num_pages=12, max_num_seqs=4, max_model_len=64, cache_of=None):
    return CacheManager(list(needs), page_size, num_pages, max_num_seqs, max_model_len, device=None, cache_of=cache_of)


def test_page_pool_is_lifo_and_refuses_double_free():
    p = PagePool(3)
    a, b = p.allocate(), p.allocate()
    assert (a, b) == (0, 1)
    p.free(a)
    assert p.allocate() == a            # the page just given back is the next one handed out
    p.free(b)
    with pytest.raises(ValueError):
        p.free(b)
    with pytest.raises(ValueError):
        p.free(7)
    p.allocate(), p.allocate()
    with pytest.raises(OutOfPages):
        p.allocate()


def test_equal_needs_share_a_group_and_different_needs_do_not():
    m = manager(needs=(WIN, FULL, WIN, FULL, None, StateCacheNeed((3, 5))))
    assert m.num_groups() == 2
    assert [m.view(i).group for i in range(4)] == [0, 1, 0, 1]
    assert m.view(0).window == 10 and m.view(1).window is None
    assert m.view(4).kind == "none" and m.view(5).kind == "state"


def test_reserve_commit_free_and_block_table():
    m = manager()
    m.add_request("a")
    m.reserve("a", 9)                    # 3 pages of 4
    assert list(m.block_table("a")[:4]) == [0, 1, 2, -1] and m.num_free_pages() == 9
    m.commit("a", 9)
    m.reserve("a", 12)                   # still 3 pages
    assert m.num_free_pages() == 9
    m.reserve("a", 13)
    assert m.block_table("a")[3] == 3
    m.commit("a", 13)
    with pytest.raises(ValueError):
        m.commit("a", 20)                # more than has pages
    m.check_invariants()
    m.free_request("a")
    assert m.num_free_pages() == 12 and not m.has_request("a")
    m.check_invariants()
    m.add_request("b")
    m.reserve("b", 4)
    assert m.block_table("b")[0] == 3    # the page freed last is used again first


def test_reserve_is_all_or_nothing():
    m = manager(num_pages=3)
    m.add_request("a")
    m.reserve("a", 8)
    m.add_request("b")
    assert not m.can_reserve("b", 8) and m.can_reserve("b", 4)
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)
    assert m.num_free_pages() == 1 and list(m.block_table("b")[:2]) == [-1, -1]
    with pytest.raises(ValueError):
        m.reserve("a", 65)               # beyond max_model_len
    m.check_invariants()


def test_window_gives_pages_back_as_it_passes_them():
    m = manager(needs=(WIN, FULL), num_pages=16)
    m.add_request("a")
    m.reserve("a", 30)
    m.commit("a", 30)
    win_table, full_table = m.block_table("a", 0), m.block_table("a", 1)
    # a query at position 30 sees keys 21..30: pages 0..4 (positions 0..19) are behind the window
    assert [int(x >= 0) for x in win_table[:8]] == [0, 0, 0, 0, 0, 1, 1, 1]
    assert all(x >= 0 for x in full_table[:8])
    assert m.num_free_pages(0) == 16 - 3 and m.num_free_pages(1) == 16 - 8
    m.check_invariants()
    for n in range(31, 45):
        m.reserve("a", n)
        m.commit("a", n)
        lo_page = max(0, n - 10 + 1) // 4
        assert all(x < 0 for x in win_table[:lo_page]) and all(x >= 0 for x in win_table[lo_page:(n + 3) // 4])
    m.check_invariants()
    m.free_request("a")
    assert m.num_free_pages(0) == 16 and m.num_free_pages(1) == 16


def test_state_slots():
    m = manager(max_num_seqs=2)
    s0, s1 = m.add_request("a"), m.add_request("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(NoFreeSlot):
        m.add_request("c")
    with pytest.raises(ValueError):
        m.add_request("a")
    m.free_request("a")
    assert m.add_request("c") == s0
    m.check_invariants()


def test_entry_reading_another_entrys_cache():
    m = manager(needs=(FULL, FULL, FULL), cache_of=[None, None, 0])
    assert m.num_groups() == 1 and len(m.groups[0].entries) == 2
    assert m.view(2).writes is False and m.view(2).group == m.view(0).group and m.view(0).writes


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    m = manager(needs=(WIN, FULL, WIN), page_size=4, num_pages=20, max_num_seqs=5, max_model_len=60)
    lengths = {}
    for it in range(600):
        op = rng.random()
        if op < 0.25 and len(lengths) < 5:
            rid = f"r{it}"
            m.add_request(rid)
            lengths[rid] = 0
        elif op < 0.85 and lengths:
            rid = rng.choice(list(lengths))
            n = lengths[rid] + rng.choice([1, 1, 1, 2, 5, 9])
            if n <= 60 and m.can_reserve(rid, n):
                m.reserve(rid, n)
                if rng.random() < 0.9:
                    m.commit(rid, n)
                    lengths[rid] = n
            elif n <= 60:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif lengths:
            rid = rng.choice(list(lengths))
            m.free_request(rid)
            del lengths[rid]
            with pytest.raises(KeyError):
                m.free_request(rid)      # freeing twice is an error, not a silent double free
        m.check_invariants()
        for rid, n in lengths.items():
            assert m.length(rid) == n
            full = m.block_table(rid, 1)
            assert all(full[i] >= 0 for i in range((n + 3) // 4))
    for rid in list(lengths):
        m.free_request(rid)
    assert m.num_free_pages(0) == 20 and m.num_free_pages(1) == 20 and m.num_free_slots() == 5


def test_a_steps_batch_arrays_are_assembled_with_slots_pages_and_checks():
    """Portions of prompts beside single decoded tokens: the flat arrays, the pages and the errors."""
    m = manager(page_size=4, num_pages=12)
    m.add_request("old")
    m.reserve("old", 6)
    m.commit("old", 6)
    tok, pos, seq_of, q_start, ctx, slots, rows, longest = m.assemble(["new", "old"], [[5, 6, 7, 8, 9], [3]], [[0, 4], [0]], vocab_size=10)
    assert list(tok) == [5, 6, 7, 8, 9, 3] and list(pos) == [0, 1, 2, 3, 4, 6] and list(seq_of) == [0, 0, 0, 0, 0, 1]
    assert list(q_start) == [0, 5, 6] and list(ctx) == [5, 7] and list(rows) == [0, 4, 5] and longest == 7
    assert list(slots) == [m.slot("new"), m.slot("old")] and m.has_request("new")
    assert (m.block_table("new")[:2] >= 0).all() and m.block_table("new")[2] == -1      # five tokens: two pages of four
    assert m.length("new") == 0 and m.length("old") == 6                                # nothing is committed yet
    m.check_invariants()
    for rids, toks, want, what in [(["old", "old"], [[1], [2]], [[], []], "twice"), (["old"], [[]], [[]], "no tokens"),
                                   (["old"], [[10]], [[0]], "vocabulary"), (["old"], [[-1]], [[0]], "vocabulary"),
                                   (["old"], [[1, 2]], [[2]], "wanted place")]:
        with pytest.raises(ValueError, match=what):
            m.assemble(rids, toks, want, vocab_size=10)
    with pytest.raises(OutOfPages):
        m.assemble(["big"], [list(range(9)) * 5], [[]], vocab_size=10)                  # 45 tokens: twelve pages, ten are free
    m.check_invariants()


def test_a_step_that_cannot_be_assembled_takes_nothing():
    """All or nothing: when a later entry of the step fails (no page, no slot, a bad token, too long),
    the entries before it have taken no slot and no page, so nothing is left reserved for a step that
    never ran."""
    m = manager(page_size=4, num_pages=6, max_num_seqs=3)
    m.add_request("old")
    m.reserve("old", 8)
    m.commit("old", 8)                                       # two pages held, four free, two slots free
    free_pages, free_slots = m.num_free_pages(), m.num_free_slots()
    bad = [(["a", "old", "b"], [[1] * 8, [2], [3] * 8], OutOfPages),                # 2 + 1 + 2 pages, four are free
           (["a", "b", "c"], [[1], [2], [3]], NoFreeSlot),                          # three new requests, two slots
           (["a", "old"], [[1, 2, 3], [10]], ValueError),                           # token outside the vocabulary
           (["a", "old"], [[1, 2, 3], [1] * 57], ValueError)]                       # beyond max_model_len (64)
    for rids, toks, error in bad:
        with pytest.raises(error):
            m.assemble(rids, toks, [[] for _ in rids], vocab_size=10)
        assert m.num_free_pages() == free_pages and m.num_free_slots() == free_slots
        assert m.live_requests() == ["old"] and m.pages_needed("old", 9) == 1
        m.check_invariants()
    m.assemble(["a", "old"], [[1] * 8, [2]], [[], [0]], vocab_size=10)              # 2 + 1 pages: fits
    assert m.num_free_pages() == free_pages - 3


def test_a_windowed_group_gets_the_pages_its_windows_need_not_the_whole_pool():
    """Two groups: one keeps every key (the pool's 200 pages), one has a window of 16 tokens.  With
    steps of at most 8 tokens and 3 live requests the windowed group's pool is 3 x (ceil(24 / 4) + 2) =
    24 pages.  Three requests run far past the window in steps of up to 8 tokens without the small
    pool ever running out, and every page comes back."""
    rng = random.Random(2)
    m = CacheManager([FULL, PagedCacheNeed(2, 16, 16)], 4, 200, 3, 256, device=None, max_step_tokens=8)
    assert m.group_pages == [200, 24] and m.spare_page(0) == 200 and m.spare_page(1) == 24
    assert m.most_tokens_alone() == 800
    lengths = {r: 0 for r in "abc"}
    for r in lengths:
        m.add_request(r)
    for _ in range(120):
        r = rng.choice("abc")
        n = rng.randint(1, 8)
        if lengths[r] + n > 256:
            continue
        m.reserve(r, lengths[r] + n)
        lengths[r] += n
        m.commit(r, lengths[r])
        m.check_invariants()
        held = sum(int((m.block_table(q, 1) >= 0).sum()) for q in lengths)
        assert held <= 24 and m.num_free_pages(1) == 24 - held
    assert max(lengths.values()) > 100
    for r in lengths:
        m.free_request(r)
    assert m.num_free_pages(0) == 200 and m.num_free_pages(1) == 24
    # without the step bound every group gets the whole pool, as before
    assert CacheManager([FULL, PagedCacheNeed(2, 16, 16)], 4, 200, 3, 256, device=None).group_pages == [200, 200]
