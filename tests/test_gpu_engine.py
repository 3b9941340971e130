"""The engine against the plain implementation, however the work is cut, in 32-bit and bfloat16."""
import numpy as np
import pytest
import torch

from helpers import (TINY, TOL, TraceBuilder, compare_trace, embed_scale_for, make_model_dir, plain_logits,
                     random_tokens, run_trace_engine)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders():
    return {name: make_model_dir(raw, seed) for name, (raw, seed) in TINY.items()}


def _requests(name, lengths, seed=11):
    raw, _ = TINY[name]
    rng = np.random.default_rng(seed)
    return {f"r{i}": random_tokens(rng, n, raw["vocab_size"]) for i, n in enumerate(lengths)}


def _plain(folder, name, requests, dtype):
    raw, _ = TINY[name]
    scale = embed_scale_for(raw, dtype)
    return {rid: plain_logits(folder, toks, embed_scale=scale) for rid, toks in requests.items()}


def _engine(folder, dtype, max_tokens):
    from kapel_b200.engine import Engine

    return Engine.from_dir(folder, dtype=dtype, max_tokens=max_tokens, max_sequences=8)


LENGTHS = {"A": [5, 17, 33, 40, 100], "B": [1, 50, 90, 200]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole(folders, name, dtype):
    """Each request alone and whole: one step, every position's logits."""
    reqs = _requests(name, LENGTHS[name])
    plain = _plain(folders[name], name, reqs, dtype)
    engine = _engine(folders[name], dtype, 256)
    tb = TraceBuilder()
    for rid, toks in reqs.items():
        tb.step([(rid, toks, range(len(toks)))], end=[rid])
    worst = compare_trace(run_trace_engine(engine, tb.steps), tb, plain, TOL[dtype], f"whole {name} {dtype}")
    print(f"whole {name} {dtype}: worst {worst:.2e}")
    engine.cache.check()
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_last_32_one_by_one(folders, name, dtype):
    """Most of a request in one step, its last 32 tokens decoded one by one."""
    reqs = _requests(name, [n for n in LENGTHS[name] if n > 32], seed=12)
    plain = _plain(folders[name], name, reqs, dtype)
    engine = _engine(folders[name], dtype, 256)
    tb = TraceBuilder()
    for rid, toks in reqs.items():
        head = len(toks) - 32
        tb.step([(rid, toks[:head], [head - 1])])
        for i in range(head, len(toks)):
            tb.step([(rid, [toks[i]], [0])], end=[rid] if i == len(toks) - 1 else [])
    worst = compare_trace(run_trace_engine(engine, tb.steps), tb, plain, TOL[dtype], f"last32 {name} {dtype}")
    print(f"last32 {name} {dtype}: worst {worst:.2e}")
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_of_changing_size(folders, name, dtype):
    """Portions of changing size, down to two tokens, every position wanted."""
    reqs = _requests(name, [LENGTHS[name][-1], LENGTHS[name][-2]], seed=13)
    plain = _plain(folders[name], name, reqs, dtype)
    engine = _engine(folders[name], dtype, 256)
    sizes = [7, 2, 13, 3, 16, 2, 31, 5, 2, 17, 64]
    tb = TraceBuilder()
    for rid, toks in reqs.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            last = at + n == len(toks)
            tb.step([(rid, toks[at : at + n], range(n))], end=[rid] if last else [])
            at += n
            k += 1
    worst = compare_trace(run_trace_engine(engine, tb.steps), tb, plain, TOL[dtype], f"portions {name} {dtype}")
    print(f"portions {name} {dtype}: worst {worst:.2e}")


def _mixed_trace(reqs, rng):
    """Up to four live requests: portions of some beside decoded tokens of others; requests are
    left out of steps now and then; a new one starts when one ends."""
    tb = TraceBuilder()
    waiting = list(reqs.items())
    live = {}                      # rid -> [tokens, fed, prompt_len]
    while waiting or live:
        while waiting and len(live) < 4:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, len(toks) - 20)]
        entries, ended = [], []
        for rid, st in list(live.items()):
            toks, fed, prompt = st
            if len(live) > 1 and rng.random() < 0.2:
                continue           # left out of this step
            if fed < prompt:
                n = min(int(rng.choice([2, 3, 5, 8, 13, 24])), prompt - fed)
                if prompt - fed - n == 1:
                    n += 1         # never leave a single prompt token: portions go down to two
                want = [n - 1]
            else:
                n, want = 1, [0]
            entries.append((rid, toks[fed : fed + n], want))
            st[1] = fed + n
            if st[1] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            tb.step(entries, end=ended)
    return tb


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_with_pages_used_again(folders, name, dtype):
    lengths = {"A": [40, 33, 17, 5, 64, 50, 21, 37, 90, 12], "B": [90, 50, 1, 33, 120, 64, 7, 100, 41, 150]}[name]
    reqs = _requests(name, lengths, seed=14)
    plain = _plain(folders[name], name, reqs, dtype)
    # Room for the four largest at once, each rounded up to 64: later requests reuse pages.
    room = sum(sorted((-(-n // 64) * 64 for n in lengths), reverse=True)[:4])
    engine = _engine(folders[name], dtype, room)
    tb = _mixed_trace(reqs, np.random.default_rng(5))
    worst = compare_trace(run_trace_engine(engine, tb.steps), tb, plain, TOL[dtype], f"mixed {name} {dtype}")
    print(f"mixed {name} {dtype}: worst {worst:.2e}, released window pages {engine.cache.released_pages}")
    engine.cache.check()
    assert engine.cache.free_pages() == engine.cache.total_pages()
    assert engine.cache.released_pages > 0
