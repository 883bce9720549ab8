"""Slots, pages and per-sequence state: nothing lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from gemmars_b200.cache import (CacheError, KVNeed, PageAllocator, SequenceCache, SlotAllocator, StateNeed)


def test_slots_are_reused_lowest_first():
    s = SlotAllocator(3)
    assert [s.take(), s.take(), s.take()] == [0, 1, 2]
    with pytest.raises(CacheError, match="no free slot"):
        s.take()
    s.give_back(1)
    with pytest.raises(CacheError, match="not held"):
        s.give_back(1)
    assert s.take() == 1 and s.held == {0, 1, 2}
    with pytest.raises(CacheError):
        s.give_back(7)


def test_pages_never_hand_out_page_zero_and_refuse_double_free():
    p = PageAllocator(4)
    got = [p.take() for _ in range(4)]
    assert sorted(got) == [1, 2, 3, 4]
    with pytest.raises(CacheError, match="full"):
        p.take()
    p.give_back(3)
    with pytest.raises(CacheError, match="not held"):
        p.give_back(3)
    assert p.take() == 3


def _cache(needs, max_tokens=64 * 6, slots=4, chunk=64, max_pos=0):
    return SequenceCache(needs, max_tokens, slots, max_pos, chunk, torch.float32, "cpu")


def test_groups_by_need_and_layout():
    full, win = KVNeed(2, 16), KVNeed(2, 16, window=40)
    c = _cache([(0, win), (1, [full]), (2, win), (4, StateNeed((3, 5)))])
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    assert (c.bindings[0][0].group, c.bindings[0][0].index) == (0, 0)
    assert (c.bindings[2][0].group, c.bindings[2][0].index) == (0, 1)
    assert c.bindings[1][0].group == 1 and c.bindings[4][0].kind == "state"
    g_win, g_full = c.kv_groups
    assert g_full.k.shape == (1, 7, 2, 64, 16) and g_win.k.shape[0] == 2
    assert g_full.table_width == 6 and g_win.table_width == (40 - 1 + 64 + 63) // 64 + 1 == 3
    assert c.state(4).shape == (5, 3, 5)


def test_an_entry_may_keep_several_things():
    """Keys with a state beside them, and two states of different shapes, for one entry; equal
    needs of different entries share a group."""
    kv, conv, s = KVNeed(2, 16), StateNeed((3, 8)), StateNeed((4, 4, 2), torch.float32)
    c = _cache([(0, [kv, conv]), (1, [s, conv]), (2, [kv])])
    assert len(c.kv_groups) == 1 and c.kv_groups[0].n_layers == 2
    assert [g.need for g in c.state_groups] == [conv, s]
    assert [(b.kind, b.group, b.index) for b in c.bindings[0]] == [("kv", 0, 0), ("state", 0, 0)]
    assert [(b.kind, b.group, b.index) for b in c.bindings[1]] == [("state", 1, 0), ("state", 0, 1)]
    v0, v1 = c.views(0), c.views(1)
    assert v0[0][0] is c.kv_groups[0] and v0[0][1].shape == (7, 2, 64, 16) and v0[1].shape == (5, 3, 8)
    assert v1[0].shape == (5, 4, 4, 2) and v1[1].shape == (5, 3, 8)
    assert v1[1].data_ptr() != v0[1].data_ptr()                  # same group, a layer of its own
    assert c.views(7) == []
    slot = c.open()
    v1[0][slot] += 1.0
    c.close(slot)
    assert c.open() == slot and float(c.views(1)[0][slot].abs().sum()) == 0.0   # cleared when the slot is taken


def test_rollback_after_a_failed_step():
    c = _cache([(0, KVNeed(1, 16))])
    s = c.open()
    c.extend(s, 70)
    held = c.pages_held()
    c.extend(s, 130)
    assert c.pages_held() == held + 2
    assert c.rollback(s, 70) is True and c.lengths[s] == 70 and c.pages_held() == held
    assert c.extend(s, 1) == 70
    # a window's ring or a state cannot be put back: the slot's length goes back, its contents may not
    w = _cache([(0, KVNeed(1, 16, window=40)), (1, StateNeed((2,)))])
    s = w.open()
    w.extend(s, 10)
    w.extend(s, 300)
    assert w.rollback(s, 10) is False and w.lengths[s] == 10
    w.close(s)
    assert w.pages_held() == 0


def test_extend_close_accounting_and_ring():
    c = _cache([(0, KVNeed(1, 16)), (1, KVNeed(1, 16, window=40))])
    full, win = c.kv_groups
    s = c.open()
    assert c.extend(s, 70) == 0 and c.lengths[s] == 70
    assert full.pages.held_count == 2 and win.pages.held_count == 2
    assert c.extend(s, 200) == 70
    assert full.pages.held_count == 5 and win.pages.held_count == 3          # the ring stops growing
    row = win.table_host[s].tolist()
    assert len(set(row)) == 3 and 0 not in row
    with pytest.raises(CacheError, match="exceeds"):
        c.extend(s, 10_000)
    assert not c.can_extend([(s, 200)])
    s2 = c.open()
    assert c.can_extend([(s2, 64)]) and not c.can_extend([(s2, 65)])
    c.close(s)
    assert full.pages.held_count == 0 and win.pages.held_count == 0 and full.table_host[s].sum() == 0
    with pytest.raises(CacheError):
        c.close(s)
    assert c.open() == s                                                   # the slot is used again


def test_truncate_and_state_clear():
    c = _cache([(0, KVNeed(1, 16)), (1, StateNeed((4,)))])
    s = c.open()
    c.extend(s, 130)
    c.state(1)[s] += 3.0
    c.truncate(s, 60)
    assert c.lengths[s] == 60 and c.kv_groups[0].pages.held_count == 1
    assert c.extend(s, 10) == 60 and c.kv_groups[0].pages.held_count == 2
    c.close(s)
    s = c.open()
    assert float(c.state(1)[s].abs().sum()) == 0.0                           # cleared when the slot is taken


def test_max_positions_bounds_a_sequence():
    c = _cache([(0, KVNeed(1, 16))], max_tokens=64 * 8, max_pos=100)
    s = c.open()
    c.extend(s, 100)
    with pytest.raises(CacheError):
        c.extend(s, 1)


def test_random_walk_keeps_the_books():
    rnd = random.Random(0)
    c = _cache([(0, KVNeed(1, 16)), (1, KVNeed(1, 16, window=70))], max_tokens=64 * 12, slots=5)
    full, win = c.kv_groups
    live = {}
    for _ in range(600):
        op = rnd.random()
        if op < 0.3 and c.slots.free_count:
            live[c.open()] = 0
        elif op < 0.8 and live:
            s = rnd.choice(list(live))
            n = rnd.randint(1, 90)
            if c.can_extend([(s, n)]):
                assert c.extend(s, n) == live[s]
                live[s] += n
        elif live:
            s = rnd.choice(list(live))
            c.close(s)
            del live[s]
        # books: pages held = pages the live sequences need; no page held twice
        want_full = sum(-(-n // 64) for n in live.values())
        assert full.pages.held_count == want_full and c.slots.held == set(live)
        pages = [int(p) for s, n in live.items() for p in full.table_host[s, :-(-n // 64)]]
        assert len(pages) == len(set(pages)) and 0 not in pages
        wpages = [int(p) for s, n in live.items() for p in win.table_host[s, :min(win.table_width, -(-n // 64))]]
        assert len(wpages) == len(set(wpages)) == win.pages.held_count and 0 not in wpages
    for s in list(live):
        c.close(s)
    assert full.pages.held_count == 0 and win.pages.held_count == 0 and c.slots.free_count == 5


def test_random_histories_lose_and_share_nothing():
    """Any order of opening, extending, truncating, rolling back and closing sequences: at every
    moment every page a table names is held by exactly one (slot, place), the held pages are the
    named ones, no page is page 0, lengths fit what is mapped, and at the end everything is back."""
    from hypothesis import given, settings, strategies as st

    ops = st.lists(st.tuples(st.sampled_from(["open", "extend", "truncate", "rollback", "close"]),
                             st.integers(0, 7), st.integers(1, 200)), min_size=1, max_size=60)

    @settings(max_examples=150, deadline=None)
    @given(ops)
    def run(history):
        c = _cache([(0, KVNeed(1, 16)), (1, KVNeed(1, 16, window=40)), (2, StateNeed((2,)))], max_tokens=64 * 10, slots=4)
        full, win = c.kv_groups
        live = []
        for op, which, n in history:
            if op == "open":
                if c.slots.free_count:
                    s = c.open()
                    assert s not in live
                    live.append(s)
                else:
                    with pytest.raises(CacheError):
                        c.open()
            elif live:
                s = live[which % len(live)]
                if op == "extend":
                    if c.can_extend([(s, n)]):
                        assert c.extend(s, n) + n == c.lengths[s]
                    else:
                        before = (c.lengths[s], c.pages_held())
                        with pytest.raises(CacheError):
                            c.extend(s, n)                       # too long, or not enough pages: nothing is taken
                        assert (c.lengths[s], c.pages_held()) == before
                elif op == "truncate":
                    keep = n % (c.lengths[s] + 1)
                    if all(g.need.window is None for g in c.kv_groups):
                        c.truncate(s, keep)
                elif op == "rollback":
                    c.rollback(s, n % (c.lengths[s] + 1))
                elif op == "close":
                    c.close(s)
                    live.remove(s)
            # ---- what must hold at every moment
            for g in (full, win):
                named = [int(p) for s in range(c.n_slots) for p in g.table_host[s].tolist() if p]
                assert len(named) == len(set(named)) == g.pages.held_count and 0 not in named
                assert g.pages.held_count + g.pages.free_count == g.pages.n
                assert int(g.table_host[c.n_slots].sum()) == 0                      # the spare row stays empty
                for s in range(c.n_slots):
                    if s not in live:
                        assert int(g.table_host[s].sum()) == 0
            for s in live:
                need = -(-c.lengths[s] // 64)
                assert sum(1 for p in full.table_host[s].tolist() if p) >= need
                assert sum(1 for p in win.table_host[s].tolist() if p) >= min(need, win.table_width)
            assert sorted(c.slots.held) == sorted(live) and set(c.lengths) == set(live)
        for s in live:
            c.close(s)
        assert c.pages_held() == 0 and c.slots.free_count == c.n_slots

    run()
