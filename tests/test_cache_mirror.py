"""The package's cache manager (bookkeeping in the C++ host library) against the plain manager of
`plain_cache.py`, driven by the same random requests: the same slots, the same pages in the same
order, the same arrays for every step, the same errors, the same free lists. No GPU needed.
"""
import numpy as np
import pytest

from kapel_b200.cache import CacheFull, CacheManager, CacheNeeds, PagedKV
from plain_cache import PlainCacheFull, PlainCacheManager


def pair(windows, pages, page_size, max_sequences):
    needs = {i: CacheNeeds(paged=PagedKV(kv_heads=2, head_dim=16 * (i + 1), window=w)) for i, w in enumerate(windows)}   # a group each
    by_needs = {needs[i].paged: pages[i] for i in range(len(windows))}
    return (CacheManager(needs, page_size, by_needs, max_sequences),
            PlainCacheManager(list(zip(windows, pages)), page_size, max_sequences))


def same_plan(a, b):
    assert a.entries == b.entries
    for name in ("positions", "row_entry", "row_count", "q_start", "q_len", "kv_len", "slots", "fresh"):
        x, y = getattr(a, name), getattr(b, name)
        assert x.dtype == y.dtype and x.shape == y.shape and np.array_equal(x, y), name
    assert len(a.groups) == len(b.groups)
    for ga, gb in zip(a.groups, b.groups):
        assert ga.lines.dtype == gb.lines.dtype == np.int32 and np.array_equal(ga.lines, gb.lines)
        assert ga.block_table.shape == gb.block_table.shape and np.array_equal(ga.block_table, gb.block_table)
        assert ga.block_table.flags["C_CONTIGUOUS"]
    assert a.taken == b.taken


def same_state(m, p):
    assert m.free_pages() == p.free_pages()
    assert m.free_slots() == p.free_slots()
    assert m.released_pages == p.released_pages
    assert sorted(m.sequences(), key=str) == sorted(p.sequences(), key=str)
    for s in m.sequences():
        assert m.length(s) == p.length(s) and m.slot(s) == p.slot(s)
        assert m.held_pages(s) == p.held_pages(s)
        for g in range(len(m.groups)):
            assert m.page_list(s, g) == list(p._sequences[s].pages[g])
    m.check()
    p.check()


@pytest.mark.parametrize("seed", range(12))
def test_the_same_requests_give_the_same_pages_arrays_and_errors(seed):
    rng = np.random.default_rng(seed)
    n_groups = int(rng.integers(1, 4))
    page_size = int(rng.choice([4, 16, 32]))
    windows = [None if rng.random() < 0.4 else int(rng.integers(1, 6 * page_size)) for _ in range(n_groups)]
    pages = [int(rng.integers(3, 30)) for _ in range(n_groups)]
    m, p = pair(windows, pages, page_size, max_sequences=int(rng.integers(1, 7)))
    next_id = 0
    for _ in range(400):
        what = rng.random()
        live = m.sequences()
        if what < 0.15 or not live:
            name = f"r{next_id}" if next_id % 2 else next_id          # ids of both kinds
            next_id += 1
            try:
                slot = m.add_sequence(name)
            except CacheFull as err:
                with pytest.raises(PlainCacheFull) as other:
                    p.add_sequence(name)
                assert (err.needed, err.free, err.group) == (other.value.needed, other.value.free, other.value.group)
            else:
                assert slot == p.add_sequence(name)
        elif what < 0.25:
            name = live[int(rng.integers(len(live)))]
            m.remove_sequence(name)
            p.remove_sequence(name)
        else:
            k = int(rng.integers(1, len(live) + 1))
            chosen = [live[i] for i in rng.permutation(len(live))[:k]]
            entries = [(s, int(rng.choice([1, 1, 1, 2, 5, 3 * page_size + 1]))) for s in chosen]
            assert m.fits(entries) == p.fits(entries)
            assert [m.pages_needed(s, c) for s, c in entries] == [p.pages_needed(s, c) for s, c in entries]
            try:
                a = m.plan(entries)
            except CacheFull as err:
                with pytest.raises(PlainCacheFull) as other:
                    p.plan(entries)
                assert (err.needed, err.free) == (other.value.needed, other.value.free)
                assert err.group.startswith(other.value.group)
            else:
                b = p.plan(entries)
                same_plan(a, b)
                if rng.random() < 0.2:
                    if rng.random() < 0.3 and len(chosen) > 1:         # one of them ends before the step is given up
                        m.remove_sequence(chosen[0])
                        p.remove_sequence(chosen[0])
                    m.abort(a)
                    p.abort(b)
                else:
                    m.commit(a)
                    p.commit(b)
        same_state(m, p)
    for s in m.sequences():
        m.remove_sequence(s)
        p.remove_sequence(s)
    same_state(m, p)
    assert m.free_pages() == m.total_pages() == pages


def test_wrong_entries_are_refused_with_the_same_errors():
    m, p = pair([None, 8], [6, 6], 4, 3)
    for c in (m, p):
        c.add_sequence("a")
        with pytest.raises(ValueError, match="twice"):
            c.plan([("a", 1), ("a", 2)])
        with pytest.raises(ValueError, match="no token"):
            c.plan([("a", 0)])
        with pytest.raises(KeyError):
            c.plan([("b", 1)])
        with pytest.raises(ValueError, match="already"):
            c.add_sequence("a")
        plan = c.plan([("a", 3)])
        c.commit(plan)
        with pytest.raises(ValueError, match="once"):
            c.commit(plan)
        with pytest.raises(ValueError, match="cannot be aborted"):
            c.abort(plan)
    same_state(m, p)
    assert m.pages_needed("nobody", 9) == p.pages_needed("nobody", 9) == [3, 3]


def test_an_empty_step_has_empty_arrays():
    m, p = pair([None], [4], 16, 2)
    same_plan(m.plan([]), p.plan([]))


def test_a_step_batch_built_from_the_plan_holds_the_plain_arrays():
    """What the engine uploads for a step (one int32 buffer, views by name) from the package's plan
    equals the plain manager's arrays; on the CPU device, so no GPU is needed."""
    import torch

    from kapel_b200.engine.batch import StepBatch

    m, p = pair([None, 24], [12, 12], 16, 4)
    for c in (m, p):
        for name in ("a", "b", "c"):
            c.add_sequence(name)
        c.commit(c.plan([("a", 40), ("b", 3)]))
    entries = [("b", 1), ("a", 30), ("c", 2)]
    a, b = m.plan(entries), p.plan(entries)
    ids = list(range(100, 100 + a.rows))
    want = [0, 5, a.rows - 1]
    batch = StepBatch(a, ids, want, torch.device("cpu"), chunk=64)
    assert batch.rows == a.rows == 33 and batch.entries == 3
    assert batch.ids.tolist() == ids and batch.want_rows.tolist() == want
    for name in ("positions", "row_entry", "row_count", "slots"):
        got = getattr(batch, name)
        assert got.dtype == torch.int32 and got.tolist() == getattr(b, name).tolist(), name
    for g, gb in zip(batch.groups, b.groups):
        assert g.lines.tolist() == gb.lines.tolist()
        assert tuple(g.block_table.shape) == gb.block_table.shape and g.block_table.tolist() == gb.block_table.tolist()
    assert batch.attention_slots(24) >= 1
    m.commit(a)
    p.commit(b)
    same_state(m, p)


def test_a_recorded_pass_s_staging_buffer_is_the_same_from_both_plans():
    """`StaticBatch.fill_host` writes a decode pass (padding rows included) into a staging buffer; the
    buffer written from the package's plan equals the one written from the plain plan. The staging
    buffers are pinned in the engine; here plain host tensors stand in, so no GPU is needed."""
    import torch

    from kapel_b200.engine.graph import StaticBatch

    m, p = pair([None, 40], [20, 20], 16, 6)
    for c in (m, p):
        for i, n in enumerate([70, 5, 33]):
            c.add_sequence(i)
            c.commit(c.plan([(i, n)]))
    entries = [(2, 1), (0, 1), (1, 1)]
    plans = m.plan(entries), p.plan(entries)
    rows, width, n_groups = 4, 8, 2                              # a bucket of four rows: one padding row
    buffers = []
    for plan in plans:
        static = StaticBatch.__new__(StaticBatch)
        static.rows, static.width, static.turn = rows, width, 0
        static.in_flight = [False, False]                        # no copy has read either buffer yet
        total = 6 * rows + n_groups * (rows + rows * width)
        static.hosts = [torch.full((total,), 12345, dtype=torch.int32) for _ in range(2)]
        assert static.fill_host(plan) == 0
        buffers.append(static.hosts[0].numpy().copy())
    assert np.array_equal(buffers[0][rows:], buffers[1][rows:])  # everything but the ids, which come later
    assert not (buffers[0][rows:] == 12345).any()                # and every word of it was written
