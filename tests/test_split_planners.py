"""How a step's attention is cut into tiles and key slots: the choices are free (they are made for
speed), but every choice must cover every key a row can see exactly once. No GPU needed.
"""
import numpy as np
import pytest

from kapel_b200.engine.batch import SPLIT_STEP, _chunks_touched, cut_tiles, decode_split, prompt_split


@pytest.mark.parametrize("window", [None, 64, 1000, 4096])
@pytest.mark.parametrize("relative", [False, True])
def test_decode_split_covers_every_visible_key(window, relative):
    rng = np.random.default_rng(3)
    for _ in range(200):
        pairs = int(rng.integers(1, 600))
        longest = int(rng.integers(1, 40000))
        sms = int(rng.choice([1, 7, 132, 148]))
        split, slots = decode_split(pairs, longest, sms, window, relative)
        assert split >= SPLIT_STEP and split % SPLIT_STEP == 0
        assert slots >= 1
        # a row of `count` keys sees [first, count); its slots are counted from key 0 or from `first`
        for count in {1, longest, max(1, longest // 2), max(1, longest - 1)}:
            first = max(0, count - window) if window else 0
            origin = first if relative else 0
            assert (count - 1 - origin) // split < slots, (pairs, longest, sms, window, relative, split, slots, count)


def test_decode_split_prefers_one_slot_when_the_pairs_fill_the_gpu():
    split, slots = decode_split(pairs=148 * 4, longest=512, sms=148)
    assert slots == 1 and split >= 512
    split, slots = decode_split(pairs=4, longest=8192, sms=148)           # few pairs, long history: many slots
    assert slots > 8 and split * slots >= 8192


@pytest.mark.parametrize("kernel", ["mma", "tcgen05", "tcgen05_pair"])
@pytest.mark.parametrize("window", [None, 300, 4096])
def test_prompt_split_covers_every_visible_key(kernel, window):
    rng = np.random.default_rng(4)
    for _ in range(100):
        tiles = int(rng.integers(1, 40))
        first = rng.integers(1, 20000, size=tiles)
        nq = rng.integers(1, 65, size=tiles)
        last = first + nq - 1
        split, slots = prompt_split(first, last, pairs_per_tile=int(rng.integers(1, 17)), sms=148, window=window,
                                    rows=int(nq.sum()), hq=8, d=int(rng.choice([64, 128, 256])), kernel=kernel)
        if slots == 1:
            assert split == 0
            continue
        assert split % SPLIT_STEP == 0 and split > 0
        assert split * slots >= int(last.max())                            # the longest row's last key has a slot
        assert split * (slots - 1) < int(last.max())                       # and no slot is empty for every row


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_pair"])
def test_prompt_split_cuts_a_few_tiles_behind_a_long_history_and_not_a_full_portion(kernel):
    """Measured on a B200 at Gemma 2 2B head sizes: 2,048 tokens behind 30,720 take 441 us uncut on
    pairs of blocks and 601 us cut into 8 slots (the tiles alone fill the GPU, and a block that
    starts among running ones costs 20 to 27 us), while one tile behind the same history is many
    times faster cut (it alone would keep one or two multiprocessors busy)."""
    per_tile = 128 if kernel == "tcgen05_pair" else 64
    for before in (4096, 30720, 129024):
        first = np.arange(before + 1, before + 2049, per_tile)
        split, slots = prompt_split(first, first + per_tile - 1, 4, 148, None, 2048, 8, 256, kernel)
        assert (split, slots) == (0, 1), (before, split, slots)
    first = np.asarray([30721])
    split, slots = prompt_split(first, first + per_tile - 1, 4, 148, None, per_tile, 8, 256, kernel)
    assert slots >= 8, (split, slots)


def test_prompt_split_of_an_empty_step_is_one_slot():
    assert prompt_split([], [], 4, 148, None, 0, 8, 256) == (0, 1)


def test_cut_tiles_keeps_every_row_once_and_in_order():
    rng = np.random.default_rng(5)
    for _ in range(100):
        n = int(rng.integers(1, 9))
        q_len = rng.integers(1, 200, size=n).astype(np.int32)
        q_start = np.concatenate([[0], np.cumsum(q_len)[:-1]]).astype(np.int32)
        per = int(rng.integers(1, 65))
        entry, row0, nq = cut_tiles(q_start, q_len, per)
        assert (nq >= 1).all() and (nq <= per).all()
        rows = np.concatenate([np.arange(r, r + k) for r, k in zip(row0, nq)])
        assert np.array_equal(rows, np.arange(int(q_len.sum())))           # every row once, ascending
        for e, r, k in zip(entry, row0, nq):                                 # a tile never crosses a request
            assert q_start[e] <= r and r + k <= q_start[e] + q_len[e]


def test_chunks_touched_counts_absolute_chunks():
    counts = np.array([1, 64, 65, 0, 1000], np.int32)
    assert _chunks_touched(counts, None, 64) == 16                          # keys 0..999 touch chunks 0..15
    assert _chunks_touched(counts, 100, 64) == 2                            # keys 900..999 touch chunks 14 and 15
    assert _chunks_touched(np.array([1025], np.int32), 100, 64) == 3        # keys 925..1024 touch chunks 14, 15 and 16
    assert _chunks_touched(np.zeros(3, np.int32), None, 64) == 1
