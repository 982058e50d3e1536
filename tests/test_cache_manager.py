"""Cache manager: no page lost, held twice or freed twice, under random orders of requests;
LIFO reuse; windowed groups give pages back as the window passes; state slots."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from slipstream_b200.cache import AllocStatus, CacheError, CacheManager, GroupLayout, OutOfPages
from slipstream_b200.parts.base import CacheSpec


def manager(pages=8, page=4, seqs=3, window=None, max_len=64, groups=None):
    layouts = groups or [GroupLayout(CacheSpec(2, 16, window), 2)]
    return CacheManager(layouts, pages, page, seqs, max_len)


def test_pages_follow_tokens_and_return_lifo():
    m = manager()
    m.admit("a")
    m.reserve("a", 5)
    assert m.get("a").tables[0] == [0, 1] and m.num_free_pages() == 6
    m.reserve("a", 5)  # already covered
    assert m.num_free_pages() == 6
    m.commit("a", 5)
    m.reserve("a", 3)  # positions 5..7 still in page 1
    assert len(m.get("a").tables[0]) == 2
    m.commit("a", 3)
    m.reserve("a", 1)
    assert m.get("a").tables[0] == [0, 1, 2]
    m.admit("b"); m.reserve("b", 1)
    m.release("a")
    m.admit("c"); m.reserve("c", 9)
    # the pages a gave back last are handed out first
    assert m.get("c").tables[0] == [0, 1, 2]
    m.check_invariants()


def test_errors():
    m = manager(pages=2)
    m.admit("a")
    with pytest.raises(OutOfPages):
        m.reserve("a", 9)
    assert m.num_free_pages() == 2  # nothing taken by the failed call
    with pytest.raises(CacheError, match="already live"):
        m.admit("a")
    with pytest.raises(CacheError, match="commit past"):
        m.commit("a", 1)
    m.release("a")
    with pytest.raises(CacheError, match="not live"):
        m.release("a")
    with pytest.raises(CacheError, match="double free"):
        m.pools[0].give_back(0, "a")
    m.admit("x"); m.admit("y"); m.admit("z")
    with pytest.raises(CacheError, match="no free state slot"):
        m.admit("w")
    big = manager(max_len=8)
    big.admit("q")
    with pytest.raises(CacheError, match="max_model_len"):
        big.reserve("q", 9)


def test_admission_status():
    m = manager(pages=4, page=4, seqs=2)
    assert m.can_admit(total_tokens=17, first_tokens=4, chunk=4) is AllocStatus.NEVER  # 5 pages > 4
    assert m.can_admit(16, 16, 16) is AllocStatus.OK
    m.admit("a"); m.reserve("a", 9)
    assert m.can_admit(8, 8, 8) is AllocStatus.LATER  # 2 pages wanted, 1 free
    assert m.can_admit(8, 4, 4) is AllocStatus.OK
    m.admit("b")
    assert m.can_admit(4, 4, 4) is AllocStatus.LATER  # no slot


def test_window_group_gives_pages_back():
    m = manager(pages=6, page=4, window=6, max_len=1000)
    m.admit("a")
    held = []
    for _ in range(40):  # 40 decode steps after nothing: never more than window/page + 2 pages
        m.reserve("a", 1); m.commit("a", 1)
        held.append(sum(1 for p in m.get("a").tables[0] if p >= 0))
        m.check_invariants()
    assert max(held) <= 3
    table = m.get("a").tables[0]
    # a query at position 40 sees keys 35..40: blocks 8, 9, 10
    assert [i for i, p in enumerate(table) if p >= 0] == [8, 9]
    assert m.peak_pages(0, 1000, 1) <= 3
    # a long portion needs pages for the window and the portion at once
    m.admit("b")
    assert m.can_admit(1000, 16, 16) is AllocStatus.NEVER or m.peak_pages(0, 1000, 16) <= 6


def test_two_groups_have_pages_of_their_own():
    groups = [GroupLayout(CacheSpec(2, 16, None), 1), GroupLayout(CacheSpec(1, 32, 4), 2)]
    m = manager(pages=5, page=2, groups=groups, max_len=100)
    m.admit("a")
    for _ in range(9):
        m.reserve("a", 1); m.commit("a", 1)
    full, win = m.get("a").tables
    assert sum(p >= 0 for p in full) == 5 and sum(p >= 0 for p in win) <= 3
    assert not m.can_reserve("a", 2)  # the full group is exhausted although the windowed one is not
    m.release("a")
    assert m.num_free_pages(0) == 5 and m.num_free_pages(1) == 5
    m.check_invariants()


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2 ** 31), st.integers(3, 12), st.sampled_from([1, 3, 4, 8]), st.sampled_from([None, 5, 16]))
def test_random_orders_keep_the_invariants(seed, pages, page, window):
    rng = random.Random(seed)
    m = manager(pages=pages, page=page, seqs=4, window=window, max_len=10 ** 6)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(300):
        op = rng.random()
        if op < 0.2 and m.num_free_slots():
            m.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 17])
            if m.can_reserve(rid, n):
                m.reserve(rid, n)
                if rng.random() < 0.9:
                    m.commit(rid, n); live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid); del live[rid]
        m.check_invariants()
        for rid, length in live.items():
            req = m.get(rid)
            assert req.length == length
            # every position a later query can see has a page
            first = 0 if window is None else max(0, length - window + 1)
            assert all(req.tables[0][b] >= 0 for b in range(first // page, (length + page - 1) // page))
    for rid in list(live):
        m.release(rid)
    assert m.num_free_pages() == pages and m.num_free_slots() == 4
    m.check_invariants()


# --------------------------------------------------------------------------- groups with pools of their own
def hybrid(full_pages=12, window_pages=3, seqs=3, max_len=128):
    layouts = [GroupLayout(CacheSpec(2, 16, None), 2), GroupLayout(CacheSpec(1, 32, 6, page_size=8), 1)]
    return CacheManager(layouts, [full_pages, window_pages], [4, 8], seqs, max_len)


def test_every_group_has_its_own_page_size_and_number_of_pages():
    m = hybrid()
    assert m.page_sizes == [4, 8] and [p.num_pages for p in m.pools] == [12, 3]
    assert [(l.page_size, l.num_pages) for l in m.groups] == [(4, 12), (8, 3)]
    m.admit("a")
    assert m.pages_needed("a", 17) == [5, 3]
    m.reserve("a", 17)
    assert m.free_pages() == [7, 0] and len(m.get("a").tables[0]) == 5 and len(m.get("a").tables[1]) == 3
    m.commit("a", 17)  # the window of 6 has left positions 0..11: the first page of 8 goes back
    assert m.free_pages() == [7, 1] and m.get("a").tables[1][0] == -1
    m.admit("b")
    # admission looks at every group: 9 tokens need 3 pages of 4 (there) and 2 pages of 8 (only 1 is free)
    assert m.can_admit(20, 9, 9) is AllocStatus.LATER
    assert m.can_admit(20, 8, 8) is AllocStatus.OK
    # never: the full group is too small for 64 tokens even when empty; the windowed group alone would cope
    assert m.can_admit(64, 4, 4) is AllocStatus.NEVER and m.peak_pages(1, 64, 4) <= 3
    assert m.can_reserve("b", 8) and not m.can_reserve("b", 9)
    m.reserve("b", 8)
    assert m.free_pages() == [5, 0]
    # together: a's next token needs nothing new, b's ninth a page of the windowed group that is not there
    assert m.can_reserve_all([("a", 1)]) and not m.can_reserve_all([("a", 1), ("b", 9)])
    m.check_invariants()
    assert 0.0 < m.utilization() <= 1.0
    m.release("a"); m.release("b")
    assert m.all_pages_free() and m.free_pages() == [12, 3]


def test_pool_sizes_give_a_windowed_group_only_what_its_windows_can_hold():
    from slipstream_b200.cache import pool_sizes, tokens_that_fit

    layouts = [GroupLayout(CacheSpec(4, 128, None), 28), GroupLayout(CacheSpec(4, 128, 1024, page_size=64), 4)]
    pools = pool_sizes(layouts, [16, 64], tokens=1 << 20, max_num_seqs=8, max_model_len=32768, max_step_tokens=2048)
    assert pools == [65536, 8 * (3072 // 64 + 1)]
    # few tokens: both follow the tokens
    assert pool_sizes(layouts, [16, 64], 1000, 8, 32768, 2048) == [63, 16]
    per_token = [28 * 2 * 4 * 128 * 2, 4 * 2 * 4 * 128 * 2]
    budget = 10 << 30
    tokens = tokens_that_fit(layouts, [16, 64], per_token, budget, 256, 32768, 2048)

    def cost(t):
        return sum(n * p * b for n, p, b in zip(pool_sizes(layouts, [16, 64], t, 256, 32768, 2048), [16, 64], per_token))

    assert cost(tokens) <= budget < cost(tokens + 64)
    # everything fits: no more than the requests can ever hold
    assert tokens_that_fit(layouts, [16, 64], per_token, 1 << 50, 4, 4096, 512) == 4 * (4096 + 64)
