"""The cache's bookkeeping (no GPU): no slot or page lost, held twice or freed twice."""
import random

import pytest

from kvad_b200.cache import CacheError, CacheFull, CacheLayout, IdPool, KVNeed, SlotBook, StateNeed
from kvad_b200.engine.batch import MetaLayout, StepEntry, pack

import numpy as np


def test_idpool_never_hands_out_twice_and_refuses_double_free():
    p = IdPool(4, "slot")
    got = [p.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        p.take()
    p.give_back(2)
    with pytest.raises(CacheError, match="not in use"):
        p.give_back(2)
    assert p.take() == 2 and p.n_free == 0


def test_grow_allocates_whole_pages_and_release_returns_all():
    b = SlotBook(3, [8], [None], page_size=64, max_positions=256)
    s = b.acquire()
    assert b.grow(s, 1) == 0 and len(b.pages[s][0]) == 1
    assert b.grow(s, 63) == 1 and len(b.pages[s][0]) == 1
    assert b.grow(s, 1) == 64 and len(b.pages[s][0]) == 2
    assert b.tokens_held() == 128
    with pytest.raises(CacheError, match="context window of 256"):
        b.grow(s, 200)
    assert b.length[s] == 65                                  # a refused step changes nothing
    b.release(s)
    b.check_all_free()
    with pytest.raises(CacheError):
        b.release(s)


def test_full_cache_refuses_without_changing_anything():
    b = SlotBook(4, [3], [None], page_size=64)
    a, c = b.acquire(), b.acquire()
    b.grow(a, 128)
    with pytest.raises(CacheFull, match="cache is full"):
        b.grow(c, 65)
    assert b.length[c] == 0 and b.pages[c][0] == [] and b.pools[0].n_free == 1
    b.grow(c, 64)
    b.release(a), b.release(c)
    b.check_all_free()


def test_random_walk_keeps_invariants():
    rnd = random.Random(0)
    b = SlotBook(6, [40, 40], [None, 100], page_size=64)
    live = []
    for _ in range(3000):
        op = rnd.random()
        if op < 0.2 and b.slots.n_free:
            live.append(b.acquire())
        elif op < 0.75 and live:
            s = rnd.choice(live)
            try:
                b.grow(s, rnd.choice([1, 1, 1, 7, 64, 130]))
                b.trim_windows(s)
            except CacheFull:
                pass
        elif live:
            s = live.pop(rnd.randrange(len(live)))
            b.release(s)
        # every page id is held by at most one (slot, group, index)
        for g, pool in enumerate(b.pools):
            held = [p for s in live for p in b.pages[s][g] if p >= 0]
            assert len(held) == len(set(held)) == pool.n_out
            assert pool.n_out + pool.n_free == pool.n
        assert sorted(live) == b.live_slots()
        for s in live:
            assert len(b.pages[s][0]) == -(-b.length[s] // 64)
    for s in live:
        b.release(s)
    b.check_all_free()


def test_window_group_drops_pages_out_of_reach():
    b = SlotBook(2, [16, 16], [None, 70], page_size=64)
    s = b.acquire()
    b.grow(s, 300)
    b.trim_windows(s)
    full, win = b.pages[s]
    assert all(p >= 0 for p in full) and len(full) == 5
    # next query at 300 reaches back to 231 = page 3; pages 0..2 are dropped
    assert [p >= 0 for p in win] == [False, False, False, True, True]
    assert b.pools[1].n_out == 2
    b.release(s)
    b.check_all_free()


def test_truncate_returns_pages():
    b = SlotBook(2, [8], [None], page_size=64)
    s = b.acquire()
    b.grow(s, 200)
    assert b.truncate(s, 70) == 70 and len(b.pages[s][0]) == 2 and b.pools[0].n_out == 2
    assert b.truncate(s, 500) == 70
    b.release(s)
    b.check_all_free()


def test_layout_groups_by_need():
    kv, win, st = KVNeed(4, 16), KVNeed(4, 16, window=32), StateNeed((8,))
    lay = CacheLayout([kv, win, kv, None, st, win])
    assert [g.entries for g in lay.groups] == [(0, 2), (1, 5), (4,)]
    assert lay.place(2) == (0, 1) and lay.place(5) == (1, 1) and lay.place(4) == (2, 0)
    assert lay.kv_groups == [0, 1] and lay.state_groups == [2]
    assert lay.bytes_per_token(2) == 2 * 4 * 4 * 16 * 2
    with pytest.raises(ValueError):
        KVNeed(0, 16)


def test_pack_rows_positions_and_wants():
    b = pack([StepEntry(7, [5, 6, 7], [0, 2]), StepEntry(2, [9], [0])], [10, 0], vocab_size=100)
    assert b.n_rows == 4 and b.n_seqs == 2 and not b.is_decode
    assert b.tokens.tolist() == [5, 6, 7, 9] and b.row_seq.tolist() == [0, 0, 0, 1]
    assert b.row_pos.tolist() == [10, 11, 12, 0] and b.seq_starts.tolist() == [0, 3, 4]
    assert b.kv_lens.tolist() == [13, 1] and b.seq_slots.tolist() == [7, 2] and b.want_rows.tolist() == [0, 2, 3]
    assert pack([StepEntry(0, [1]), StepEntry(1, [2])], [4, 9], 10).is_decode
    for bad in ([StepEntry(0, [], [])], [StepEntry(0, [100])], [StepEntry(0, [1], [1])],
                [StepEntry(0, [1]), StepEntry(0, [2])], []):
        with pytest.raises(ValueError):
            pack(bad, [0] * len(bad), 100)


def test_meta_layout_sections_do_not_overlap():
    lay = MetaLayout(16, 4, {0: 3, 1: 5})
    host = np.full(lay.total, -7, dtype=np.int32)
    b = pack([StepEntry(1, [5, 6, 7], [2]), StepEntry(3, [9, 9], [1])], [0, 64], 100)
    lay.fill(host, b, {0: [[11], [12, 13]], 1: [[21], [22, 23]]})
    assert host[lay.tokens:lay.tokens + 5].tolist() == [5, 6, 7, 9, 9]
    assert host[lay.row_pos:lay.row_pos + 5].tolist() == [0, 1, 2, 64, 65]
    assert host[lay.tables[0]:lay.tables[0] + 6].tolist() == [11, -7, -7, 12, 13, -7]
    assert host[lay.tables[1] + 5:lay.tables[1] + 7].tolist() == [22, 23]
    starts = sorted([lay.tokens, lay.row_seq, lay.row_pos, lay.seq_starts, lay.kv_lens, lay.seq_slots,
                     lay.want_rows, *lay.tables.values()])
    assert len(set(starts)) == len(starts) and all(s % 4 == 0 for s in starts)
