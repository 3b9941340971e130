"""The cache manager: pages by layer group, block tables, window release, slots, random orders."""
import numpy as np
import pytest

from kapel_b200.cache import CacheFull, CacheManager, CacheNeeds, PagedKV, PagePool, StateSpec


def manager(pages=8, window=24, max_sequences=4):
    needs = {0: CacheNeeds(PagedKV(2, 16, window)), 1: CacheNeeds(PagedKV(2, 16, None)), 2: CacheNeeds(PagedKV(2, 16, window))}
    return CacheManager(needs, 16, pages, max_sequences)


def test_pool_takes_and_gives_whole_pages():
    pool = PagePool(3)
    a, b = pool.take(), pool.take()
    assert (a, b) == (0, 1) and pool.free == 1
    pool.give(a)
    assert pool.take() == a                      # the page freed last is taken first
    with pytest.raises(ValueError, match="twice"):
        pool.give(2)
    pool.take()
    with pytest.raises(CacheFull):
        pool.take()
    with pytest.raises(ValueError, match="not of this pool"):
        pool.give(7)
    pool.check()


def test_layers_with_the_same_needs_share_a_group():
    m = manager()
    assert len(m.groups) == 2
    assert m.group_of_layer == {0: 0, 1: 1, 2: 0}
    assert [g.window for g in m.groups] == [24, None]


def test_a_step_describes_its_rows():
    m = manager()
    m.add_sequence("a")
    m.add_sequence("b")
    p = m.plan([("a", 20), ("b", 3)])
    assert p.rows == 23
    assert p.positions.tolist() == list(range(20)) + [0, 1, 2]
    assert p.row_entry.tolist() == [0] * 20 + [1] * 3
    assert p.row_count.tolist() == list(range(1, 21)) + [1, 2, 3]
    assert p.q_start.tolist() == [0, 20] and p.q_len.tolist() == [20, 3] and p.kv_len.tolist() == [20, 3]
    assert p.fresh.tolist() == [True, True] and sorted(p.slots.tolist()) == [1, 2]
    for g in p.groups:
        table = g.block_table
        assert table.shape == (2, 2) and table[1, 1] == -1
        lines = g.lines.tolist()
        assert len(set(lines)) == 23, "two rows write one line"
        assert lines[:16] == [table[0, 0] * 16 + i for i in range(16)]
        assert lines[16:20] == [table[0, 1] * 16 + i for i in range(4)]
    assert m.length("a") == 0, "lengths move at commit"
    m.commit(p)
    assert m.length("a") == 20 and m.length("b") == 3
    p2 = m.plan([("b", 1)])
    assert p2.positions.tolist() == [3] and p2.row_count.tolist() == [4] and p2.fresh.tolist() == [False]
    assert p2.taken == []                        # the token fits its page
    m.commit(p2)
    m.check()


def test_refusals_take_nothing():
    m = manager(pages=2)
    m.add_sequence("a")
    with pytest.raises(ValueError, match="twice"):
        m.plan([("a", 1), ("a", 1)])
    with pytest.raises(ValueError, match="no token"):
        m.plan([("a", 0)])
    with pytest.raises(KeyError):
        m.plan([("zz", 1)])
    with pytest.raises(CacheFull) as info:
        m.plan([("a", 33)])
    assert (info.value.needed, info.value.free) == (3, 2)
    assert m.free_pages() == [2, 2]
    assert m.pages_needed("a", 33) == [3, 3] and m.fits([("a", 32)]) and not m.fits([("a", 33)])
    with pytest.raises(ValueError, match="already"):
        m.add_sequence("a")


def test_abort_gives_back_what_the_plan_took():
    m = manager()
    m.add_sequence("a")
    m.commit(m.plan([("a", 10)]))
    before = m.free_pages()
    p = m.plan([("a", 40)])
    assert m.free_pages() == [before[0] - 3, before[1] - 3]
    m.abort(p)
    assert m.free_pages() == before and m.length("a") == 10
    m.check()
    with pytest.raises(ValueError):
        m.commit(p)


def test_a_window_gives_back_the_pages_it_has_passed():
    m = manager(pages=8, window=24)
    m.add_sequence("a")
    m.commit(m.plan([("a", 40)]))
    # length 40: the next query has seen 41 and reads from 17 on; page 0 (positions 0..15) is done.
    assert m.held_pages("a") == [2, 3]
    m.commit(m.plan([("a", 16)]))
    # length 56: reads from 33 on; pages 0 and 1 are done.
    assert m.held_pages("a") == [2, 4]
    p = m.plan([("a", 1)])
    assert p.groups[0].block_table[0].tolist()[:2] == [-1, -1] and p.groups[0].block_table[0, 2] >= 0
    assert (p.groups[1].block_table[0] >= 0).all()
    m.commit(p)
    assert m.released_pages == 2
    m.remove_sequence("a")
    assert m.free_pages() == [8, 8]
    m.check()


def test_a_long_sequence_lives_in_a_small_windowed_pool():
    needs = {0: CacheNeeds(PagedKV(1, 16, 32))}
    m = CacheManager(needs, 16, 4, 2)           # 64 positions of pages for a sequence of 400
    m.add_sequence("a")
    m.commit(m.plan([("a", 30)]))
    for _ in range(370):
        m.commit(m.plan([("a", 1)]))
        m.check()
    assert m.length("a") == 400 and m.held_pages("a")[0] <= 3


def test_slots_and_fresh():
    needs = {0: CacheNeeds(state=StateSpec((4,))), 1: CacheNeeds(PagedKV(1, 16))}
    made = []
    m = CacheManager(needs, 16, 4, 2, allocate=lambda shape, dtype: made.append((shape, dtype)) or object(), dtype="bf16")
    assert ((3, 4), "float32") in made and ((4, 1, 16, 16), "bf16") in made
    a, b = m.add_sequence("a"), m.add_sequence("b")
    assert {a, b} == {1, 2}
    with pytest.raises(CacheFull):
        m.add_sequence("c")
    m.remove_sequence("a")
    assert m.add_sequence("c") == a
    m.check()


def test_random_orders_lose_no_page_and_hold_none_twice():
    rng = np.random.default_rng(0)
    for trial in range(20):
        m = manager(pages=int(rng.integers(6, 20)), window=int(rng.choice([16, 24, 40])), max_sequences=5)
        live, next_id = {}, 0
        for _ in range(300):
            r = rng.random()
            if (r < 0.2 or not live) and len(live) < 5:
                m.add_sequence(next_id)
                live[next_id] = 0
                next_id += 1
            elif r < 0.35:
                victim = int(rng.choice(list(live)))
                m.remove_sequence(victim)
                del live[victim]
            else:
                chosen = [s for s in live if rng.random() < 0.6] or [next(iter(live))]
                entries = [(s, int(rng.choice([1, 1, 1, 2, 7, 16, 33]))) for s in chosen]
                try:
                    p = m.plan(entries)
                except CacheFull:
                    m.check()
                    continue
                lines = np.concatenate([p.groups[0].lines, ])
                assert len(set(lines.tolist())) == len(lines)
                if rng.random() < 0.1:
                    m.abort(p)
                else:
                    m.commit(p)
                    for s, c in entries:
                        live[s] += c
            m.check()
            for s, n in live.items():
                assert m.length(s) == n
        for s in list(live):
            m.remove_sequence(s)
        m.check()
        assert m.free_pages() == m.total_pages() and m.free_slots() == 5
