"""The cache manager on the host: no page lost, held twice or freed twice, under random orders."""

import random

import numpy as np
import pytest

from jax_llm_examples_b200.cache import CacheError, CacheManager, OutOfPages, OutOfSlots, Retention


def _manager(page=16, slots=4, width=32, pages=24, chunk=32, window=None):
    m = CacheManager(page, slots, width)
    m.add_group(Retention.all(), pages)
    m.add_group(Retention.chunk(chunk), pages)
    if window:
        m.add_group(Retention.window(window), pages)
    return m


def test_reserve_commit_release_counts():
    m = _manager()
    s = m.alloc_slot()
    assert m.pages_needed(s, 40) == 3
    m.reserve(s, 40)
    assert m.free_pages(0) == 21 and m.free_pages(1) == 21
    assert m.commit(s, 40) == 2  # chunk group: positions < 32 are dead -> pages 0 and 1
    assert m.pages_held(s, 0) == 3 and m.pages_held(s, 1) == 1
    assert list(m.table(1)[s][:3]) == [-1, -1, m.table(1)[s][2]] and m.table(1)[s][2] >= 0
    m.reserve(s, 70)
    m.commit(s, 70)  # chunk starts at 64 -> pages 2, 3 dead
    assert m.pages_held(s, 1) == 1 and m.pages_held(s, 0) == 5
    m.check()
    assert m.release(s) == 6
    assert m.free_pages(0) == 24 and m.free_pages(1) == 24 and m.free_slots() == 4
    m.check()


def test_chunk_pages_stay_while_a_portion_straddles_the_boundary():
    m = _manager()
    s = m.alloc_slot()
    m.reserve(s, 30)
    m.commit(s, 30)
    m.reserve(s, 45)  # a portion from 30 to 44 crosses the chunk start 32: the old chunk's pages must be there
    assert m.pages_held(s, 1) == 3
    assert all(p >= 0 for p in m.table(1)[s][:3])
    assert m.commit(s, 45) == 2
    m.check()


def test_page_not_dividing_the_chunk_keeps_the_straddling_page():
    m = CacheManager(16, 2, 16)
    m.add_group(Retention.chunk(40), 8)
    s = m.alloc_slot()
    m.reserve(s, 50)
    assert m.commit(s, 50) == 2  # chunk starts at 40; page 2 (32..47) holds 40..47 and stays
    assert list(m.table(0)[s][:4] >= 0) == [False, False, True, True]


def test_window_group_releases_behind_the_window():
    m = _manager(window=20)
    s = m.alloc_slot()
    m.reserve(s, 100)
    m.commit(s, 100)  # next query at 100 reads keys >= 81 -> pages 0..4 (positions < 80) are dead
    assert m.pages_held(s, 2) == 2 and m.pages_held(s, 0) == 7
    m.check()


def test_out_of_pages_takes_nothing_and_pages_are_reused_lifo():
    m = _manager(pages=4)
    a, b = m.alloc_slot(), m.alloc_slot()
    m.reserve(a, 48)
    with pytest.raises(OutOfPages):
        m.reserve(b, 33)
    assert m.free_pages(0) == 1 and m.reserved(b) == 0
    m.check()
    held = set(int(p) for p in m.table(0)[a][:3])
    m.release(a)
    m.reserve(b, 48)
    assert set(int(p) for p in m.table(0)[b][:3]) == held  # the pages given back are handed out again
    m.check()


def test_misuse_is_refused():
    m = _manager()
    s = m.alloc_slot()
    m.reserve(s, 10)
    with pytest.raises(CacheError, match="cannot commit"):
        m.commit(s, 11)
    m.commit(s, 10)
    with pytest.raises(CacheError, match="cannot commit"):
        m.commit(s, 5)
    with pytest.raises(CacheError, match="exceeds the block table"):
        m.reserve(s, 16 * 32 + 1)
    m.release(s)
    with pytest.raises(CacheError, match="released twice"):
        m.release(s)
    with pytest.raises(CacheError):
        m.reserve(s, 20)
    for _ in range(4):
        m.alloc_slot()
    with pytest.raises(OutOfSlots):
        m.alloc_slot()
    with pytest.raises(CacheError):
        CacheManager(0, 1, 1)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    page, pages, chunk = rng.choice([4, 16, 64]), rng.choice([8, 24, 60]), rng.choice([24, 32, 100])
    m = CacheManager(page, 5, 64)
    m.add_group(Retention.all(), pages)
    m.add_group(Retention.chunk(chunk), pages)
    m.add_group(Retention.window(rng.choice([5, 40])), pages)
    live: dict[int, int] = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.15 and len(live) < 5:
            live[m.alloc_slot()] = 0
        elif op < 0.3 and live:
            s = rng.choice(list(live))
            m.release(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 33])
            if (live[s] + n + page - 1) // page > 64:
                continue
            try:
                m.reserve(s, live[s] + n)
            except OutOfPages:
                assert m.reserved(s) == max(live[s], m.reserved(s))
                m.check()
                continue
            if rng.random() < 0.9:
                live[s] += n
                m.commit(s, live[s])
                # what the next query can read is all there
                for g, r in enumerate(m.groups):
                    first = 0 if r.kind == 0 else ((live[s] // r.size) * r.size if r.kind == 1 else max(0, live[s] - r.size + 1))
                    row = m.table(g)[s]
                    assert all(row[i] >= 0 for i in range(first // page, (live[s] + page - 1) // page))
        m.check()
    for s in list(live):
        m.release(s)
    m.check()
    assert all(m.free_pages(g) == pages for g in range(3)) and m.free_slots() == 5


def test_pack_step_layout():
    m = _manager(page=4, slots=3, width=8, pages=10, chunk=8)
    a, b = m.alloc_slot(), m.alloc_slot()
    m.reserve(a, 5)
    m.commit(a, 5)
    m.reserve(a, 6)
    m.reserve(b, 3)
    out = np.zeros(CacheManager.packed_size(2, 4, 2, 3, 2), dtype=np.int32)
    n = m.pack_step(np.array([a, b], np.int32), np.array([1, 3], np.int32), np.array([9, 5, 6, 7], np.int32),
                    np.array([0, 1, 3], np.int32), np.array([0, 0, 2], np.int32), 2, 4, 2, 3, out)
    assert n == out.size
    tok, pos, req = out[0:4], out[4:8], out[8:12]
    cu, start, kv, slots, rows = out[12:15], out[15:17], out[17:19], out[19:21], out[21:24]
    assert list(tok) == [9, 5, 6, 7] and list(pos) == [5, 0, 1, 2] and list(req) == [0, 1, 1, 1]
    assert list(cu) == [0, 1, 4] and list(start) == [5, 0] and list(kv) == [6, 3] and list(slots) == [a, b]
    assert list(rows) == [0, 1, 3]
    tables = out[24:].reshape(2, 2, 2)
    assert np.array_equal(tables[0][0], m.table(0)[a][:2]) and np.array_equal(tables[1][1], m.table(1)[b][:2])
    with pytest.raises(CacheError, match="not reserved"):
        m.pack_step(np.array([a], np.int32), np.array([5], np.int32), np.zeros(5, np.int32), np.array([0, 0], np.int32),
                    np.zeros(0, np.int32), 8, 5, 1, 0, np.zeros(200, np.int32))
    with pytest.raises(CacheError, match="wanted place"):
        m.pack_step(np.array([a], np.int32), np.array([1], np.int32), np.zeros(1, np.int32), np.array([0, 1], np.int32),
                    np.array([1], np.int32), 8, 1, 1, 1, np.zeros(200, np.int32))
