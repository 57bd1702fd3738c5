"""The cache's bookkeeping (the library's, cache/cache.cpp) on the host: no page or
slot is lost, held twice or freed twice; window groups give pages back; a refused
step changes nothing.  The two tests of per-sequence state need the device."""
import numpy as np
import pytest
import torch

from janas_b200.cache import PAGE, Cache, CacheFull, KVSpec, PagePool, SlotPool, StateSpec


def test_page_pool():
    p = PagePool(4)
    a = p.take(3)
    assert sorted(a) == [0, 1, 2] and p.n_free == 1
    with pytest.raises(CacheFull):
        p.take(2)
    assert p.n_free == 1                       # a refused take takes nothing
    p.give_back(a[:1])
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back(a[:1])                     # freed twice
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back([3])                       # never handed out
    p.check()
    b = p.take(2)
    assert set(b) & set(a[1:]) == set()        # held pages are not handed out again
    p.check()


def test_slot_pool():
    s = SlotPool(2)
    a, b = s.take(), s.take()
    assert a != b
    with pytest.raises(CacheFull):
        s.take()
    s.give_back(a)
    with pytest.raises(RuntimeError):
        s.give_back(a)
    assert s.take() == a                       # a freed slot is used again
    s.check()


def make(max_tokens=512, max_seqs=4, window=0, state=False):
    kv = [KVSpec(2, 16), KVSpec(2, 16), KVSpec(1, 32, window) if window else KVSpec(2, 16), None]
    st = [None, StateSpec((3,)) if state else None, None, None]
    return Cache(kv, st, max_tokens, max_seqs, torch.float32, "cuda:0" if state else "cpu")


def test_groups_have_storage_of_their_own():
    c = make(window=100)
    assert len(c.groups) == 2
    full, win = c.groups
    assert full.entries == [0, 1] and win.entries == [2]
    assert full.k.shape == (2, 8, 2, PAGE, 16) and win.k.shape == (1, 8, 1, PAGE, 32)
    assert 3 not in c.group_of


def test_reserve_advance_free():
    c = make()
    a, b = c.new_sequence(), c.new_sequence()
    c.reserve([a, b], [70, 1])
    c.advance([a, b], [70, 1])
    g = c.groups[0]
    assert g.held(a) == 2 and g.held(b) == 1 and c.tokens_held() == 3 * PAGE
    bt = c.block_table(g, [b, a])
    assert bt.shape == (2, 8) and bt.dtype == np.int32
    assert bt[0, 0] == g.pages[b][0] and list(bt[1, :2]) == g.pages[a] and bt[1, 2] == -1
    for _ in range(58):                         # a grows to 128: still two pages
        c.reserve([a], [1]); c.advance([a], [1])
    assert g.held(a) == 2
    c.reserve([a], [1]); c.advance([a], [1])
    assert g.held(a) == 3 and c.length[a] == 129
    c.check()
    c.free_sequence(a)
    with pytest.raises(RuntimeError):
        c.free_sequence(a)
    c.free_sequence(b)
    c.check()
    assert c.tokens_held() == 0


def test_full_cache_refuses_the_whole_step():
    c = make(max_tokens=256)
    a, b = c.new_sequence(), c.new_sequence()
    c.reserve([a], [100]); c.advance([a], [100])
    before = (c.groups[0].pool.n_free, list(c.groups[0].pages[a]), list(c.groups[0].pages[b]))
    with pytest.raises(CacheFull):
        c.reserve([a, b], [20, 129])            # a would fit, b not: neither is taken
    assert (c.groups[0].pool.n_free, c.groups[0].pages[a], c.groups[0].pages[b]) == before
    c.check()


def test_window_group_gives_pages_back():
    c = make(max_tokens=1024, window=100)
    full, win = c.groups
    s = c.new_sequence()
    c.reserve([s], [300]); c.advance([s], [300])
    assert full.held(s) == 5
    # the token at 300 sees 201..300: pages 3 and 4; pages 0..2 are gone
    assert win.pages[s][:3] == [-1, -1, -1] and win.held(s) == 2
    for _ in range(100):
        c.reserve([s], [1]); c.advance([s], [1])
    assert full.held(s) == 7 and win.held(s) <= 3
    c.check()
    c.free_sequence(s)
    c.check()
    assert win.pool.n_free == win.pool.n_pages and full.pool.n_free == full.pool.n_pages


@pytest.mark.gpu
def test_state_is_zero_for_a_new_sequence():
    c = make(state=True)
    s = c.new_sequence()
    c.mixer_state[1][s] += 5.0
    c.free_sequence(s)
    t = c.new_sequence()
    torch.cuda.synchronize()
    assert t == s and float(c.mixer_state[1][t].abs().sum()) == 0.0


def test_many_sequences_come_and_go():
    rng = np.random.default_rng(0)
    c = make(max_tokens=64 * 40, max_seqs=6, window=90)
    live = {}
    for it in range(400):
        if live and (rng.random() < 0.3 or len(live) == 6):
            s = list(live)[int(rng.integers(len(live)))]
            c.free_sequence(s)
            del live[s]
        elif len(live) < 6 and rng.random() < 0.5:
            s = c.new_sequence()
            n = int(rng.integers(1, 200))
            try:
                c.reserve([s], [n]); c.advance([s], [n]); live[s] = n
            except CacheFull:
                c.free_sequence(s)
        elif live and rng.random() < 0.25:
            # a sequence goes back: part of the way where the window group still holds
            # what the token at that place sees, else not at all (and nothing changes)
            s = list(live)[int(rng.integers(len(live)))]
            n = int(rng.integers(0, live[s] + 1))
            could = c.can_truncate(s, n)
            assert c.truncate(s, n) == could
            if could:
                live[s] = n
            win = c.groups[1]
            first = win.first_needed_page(live[s])
            assert all(p >= 0 for p in win.pages[s][first:])     # what the next token sees is held
        elif live:
            ss = list(live)
            try:
                c.reserve(ss, [1] * len(ss)); c.advance(ss, [1] * len(ss))
                for s in ss:
                    live[s] += 1
            except CacheFull:
                pass
        c.check()
        for s, n in live.items():
            assert c.length[s] == n and c.groups[0].held(s) == (n + PAGE - 1) // PAGE
    for s in list(live):
        c.free_sequence(s)
    c.check()
    assert c.tokens_held() == 0


def test_truncate_gives_pages_back_and_knows_what_cannot_be_undone():
    c = make(max_tokens=1024, window=100)
    full, win = c.groups
    s = c.new_sequence()
    c.reserve([s], [300]); c.advance([s], [300])
    assert not c.truncate(s, 301) and not c.truncate(s, -1)
    assert c.truncate(s, 300)                           # nothing to do
    # a token at 250 would see 151..250: page 2, which the window group gave back
    assert not c.can_truncate(s, 250) and not c.truncate(s, 250)
    assert int(c.length[s]) == 300 and full.held(s) == 5
    # a token at 290 sees 191..290, which begins in page 2 as well
    assert not c.truncate(s, 290)
    # a token at 299 sees 200..299: pages 3 and 4, both held
    assert c.truncate(s, 299) and int(c.length[s]) == 299
    c.check()
    assert c.truncate(s, 0)
    assert int(c.length[s]) == 0 and full.held(s) == 0 and win.held(s) == 0
    c.check()
    c.reserve([s], [70]); c.advance([s], [70])
    assert c.truncate(s, 10) and full.held(s) == 1 and win.held(s) == 1
    c.reserve([s], [200]); c.advance([s], [200])
    c.check()
    c.free_sequence(s)
    c.check()
    assert win.pool.n_free == win.pool.n_pages and full.pool.n_free == full.pool.n_pages


@pytest.mark.gpu
def test_truncate_with_a_state_of_fixed_size_goes_back_to_nothing_only():
    c = make(state=True)
    s = c.new_sequence()
    c.reserve([s], [20]); c.advance([s], [20])
    c.mixer_state[1][s] += 5.0
    assert not c.truncate(s, 10) and int(c.length[s]) == 20
    assert float(c.mixer_state[1][s].abs().sum()) > 0
    assert c.truncate(s, 0)
    assert float(c.mixer_state[1][s].abs().sum()) == 0.0      # as for a new sequence
    c.free_sequence(s)
    c.check()
