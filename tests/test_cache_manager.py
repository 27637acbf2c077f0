"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders
of requests; windowed groups give pages back as the window passes; state slots are zeroed."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from hfee_b200.cache import CacheManager, FixedState, OutOfPages, PagedKV, PagePool


def manager(num_pages=8, page=4, reqs=3, ctx=64, needs=None):
    needs = needs or {0: PagedKV(2, 8), 1: PagedKV(2, 8)}
    return CacheManager(needs, page, num_pages, reqs, ctx, torch.float32, "cpu")


def test_page_pool_refuses_double_free_and_overdraw():
    p = PagePool(3)
    a = p.take(2)
    assert a == [0, 1] and p.free_pages == 1
    with pytest.raises(OutOfPages):
        p.take(2)
    assert p.free_pages == 1                       # nothing was taken
    p.give_back([1])
    with pytest.raises(ValueError, match="twice"):
        p.give_back([1])
    assert p.take(1) == [1]                        # the page freed last is reused first


def test_reserve_is_all_or_nothing_and_close_returns_everything():
    m = manager(num_pages=5)
    a, b = m.open(), m.open()
    m.reserve(a, 9); m.commit(a, 9)                # 3 pages
    assert m.free_pages() == 2
    with pytest.raises(OutOfPages):
        m.reserve(b, 13)                           # needs 4
    assert m.free_pages() == 2 and not m.can_reserve(b, 9) and m.can_reserve(b, 8)
    m.reserve(b, 8); m.commit(b, 5)
    m.reserve(b, 8)                                # already covered: takes nothing
    assert m.free_pages() == 0
    m.check_invariants()
    m.close(a)
    assert m.free_pages() == 3
    m.check_invariants()
    with pytest.raises(ValueError, match="not open"):
        m.close(a)
    c = m.open()
    assert c == a and m.length[c] == 0
    m.reserve(c, 4)
    assert int(m.paged[0].table[c, 0]) >= 0 and int(m.paged[0].table[c, 1]) == -1
    with pytest.raises(ValueError, match="context limit"):
        m.reserve(c, 65)


def test_groups_by_need_and_views():
    needs = {0: PagedKV(2, 8), 1: PagedKV(2, 8), 2: PagedKV(1, 16, window=6), 3: FixedState((5,), "float32"), 4: None}
    m = manager(needs=needs)
    assert len(m.paged) == 2 and len(m.states) == 1
    assert m.view(0).k.shape == (8, 2, 4, 8) and m.view(2).k.shape == (8, 1, 4, 16)
    assert m.view(0).block_table is m.view(1).block_table and m.view(0).k.data_ptr() != m.view(1).k.data_ptr()
    assert m.view(3).state.shape == (3, 5) and m.view(4) is None
    with pytest.raises(TypeError):
        manager(needs={0: "pages please"})


def test_window_gives_pages_back_as_it_passes():
    m = manager(num_pages=6, page=4, needs={0: PagedKV(1, 8, window=6)})
    s = m.open()
    held = []
    for n in range(1, 41):
        m.reserve(s, n); m.commit(s, n)
        m.check_invariants()
        row = m.paged[0].table[s]
        held.append(int((row >= 0).sum()))
        first_key = max(0, n - 6 + 1)              # lowest key the next token (position n) reads
        assert all(row[p] >= 0 for p in range(first_key // 4, -(-n // 4)))
        assert all(row[p] < 0 for p in range(0, first_key // 4))
    assert max(held) <= 3 and m.free_pages() >= 3  # 40 tokens passed through at most 3 live pages
    m.close(s)
    assert m.free_pages() == 6


def test_state_rows_are_zeroed_at_admission():
    m = manager(needs={0: FixedState((4,), "float32")})
    s = m.open()
    m.view(0).state[s] += 3.0
    m.close(s)
    assert m.open() == s and float(m.view(0).state[s].abs().sum()) == 0.0


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["open", "grow", "close"]), st.integers(0, 5), st.integers(1, 23)),
                min_size=1, max_size=80), st.sampled_from([None, 5, 9]))
def test_random_orders_keep_every_page_accounted_for(ops_list, window):
    m = manager(num_pages=10, page=4, reqs=4, ctx=48, needs={0: PagedKV(1, 8), 1: PagedKV(1, 8, window=window)})
    live = []
    for op, pick, n in ops_list:
        if op == "open" and m.free_slots():
            live.append(m.open())
        elif op == "grow" and live:
            s = live[pick % len(live)]
            want = min(m.length[s] + n, 48)
            if m.can_reserve(s, want):
                before = m.free_pages()
                m.reserve(s, want)
                m.commit(s, want)
                assert m.free_pages() <= before or window is not None
            else:
                before = [g.pool.free_pages for g in m.paged]
                with pytest.raises(OutOfPages):
                    m.reserve(s, want)
                assert before == [g.pool.free_pages for g in m.paged]
        elif op == "close" and live:
            m.close(live.pop(pick % len(live)))
        m.check_invariants()
    for s in live:
        m.close(s)
    m.check_invariants()
    assert all(g.pool.free_pages == 10 for g in m.paged)
