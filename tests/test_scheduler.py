"""The scheduler's decisions, on the CPU, over a stand-in engine with a real cache manager."""
import numpy as np
import pytest

from kapel_b200.cache import CacheManager, CacheNeeds, PagedKV
from kapel_b200.engine.scheduler import EngineOptions, Request, Scheduler
from kapel_b200.sampling import Sampling

VOCAB = 50


class FakeEngine:
    """Logits that depend only on the request's tokens so far: next = (sum of tokens * 7 + count) % VOCAB.
    It keeps what it was fed per request, as the cache would, so a cut or a recomputation that
    loses or repeats a token shows as a wrong next token."""

    def __init__(self, pages=8, window=None, max_sequences=8):
        needs = {0: CacheNeeds(PagedKV(1, 16, None))}
        if window:
            needs[1] = CacheNeeds(PagedKV(1, 16, window))
        self.cache = CacheManager(needs, 16, pages, max_sequences)
        self.vocab_size = VOCAB
        self.fed = {}
        self.passes = []

    @staticmethod
    def next_token(tokens):
        return (sum(tokens) * 7 + len(tokens)) % VOCAB

    def step(self, entries):
        counts = []
        for e in entries:
            if e.id not in self.cache:
                raise AssertionError("the scheduler admits before it steps")
            counts.append((e.id, len(e.tokens)))
        plan = self.cache.plan(counts)
        rows = []
        for e in entries:
            self.fed.setdefault(e.id, []).extend(e.tokens)
            assert len(self.fed[e.id]) == self.cache.length(e.id) + len(e.tokens)
            for w in e.want:
                assert w == len(e.tokens) - 1
                row = np.full(VOCAB, -5.0)
                row[self.next_token(self.fed[e.id])] = 5.0
                rows.append(row)
        self.cache.commit(plan)
        self.passes.append([(e.id, len(e.tokens)) for e in entries])
        return np.array(rows).reshape(-1, VOCAB)

    def end(self, seq_id):
        if seq_id in self.cache:
            self.cache.remove_sequence(seq_id)
        self.fed.pop(seq_id, None)


class StagingEngine(FakeEngine):
    """The stand-in with the three calls that let the scheduler stage a decode pass ahead."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.staged = self.ran_staged = self.discarded = 0

    def prepare_decode(self, seq_ids):
        from kapel_b200.cache import CacheFull

        try:
            plan = self.cache.plan([(s, 1) for s in seq_ids])
        except CacheFull:
            return None
        self.staged += 1
        return (plan, list(seq_ids))

    def step_prepared(self, handle, ids):
        plan, seq_ids = handle
        rows = []
        for s, t in zip(seq_ids, ids):
            self.fed[s].append(t)
            assert len(self.fed[s]) == self.cache.length(s) + 1
            row = np.full(VOCAB, -5.0)
            row[self.next_token(self.fed[s])] = 5.0
            rows.append(row)
        self.cache.commit(plan)
        self.passes.append([(s, 1) for s in seq_ids])
        self.ran_staged += 1
        return np.array(rows).reshape(-1, VOCAB)

    def discard(self, handle):
        if not handle[0].committed:
            self.cache.abort(handle[0])
            self.discarded += 1


def expected(prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(FakeEngine.next_token(seq))
    return seq[len(prompt):]


def run(sched, limit=10000):
    out = {}
    finishes = {}
    for _ in range(limit):
        if not sched.has_work():
            break
        for ev in sched.step():
            if ev.token is not None:
                out.setdefault(ev.id, []).append(ev.token)
            if ev.finish:
                finishes[ev.id] = (ev.finish, ev.error)
    assert not sched.has_work(), "the scheduler did not finish"
    return out, finishes


def prompts(rng, lengths):
    return [[int(t) for t in rng.integers(0, VOCAB, size=n)] for n in lengths]


def test_a_staged_pass_runs_if_nothing_changed_and_gives_its_pages_back_if_something_did():
    eng = StagingEngine(pages=64)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=64))
    a, b = [3, 9, 27, 4], [5] * 20
    eos = expected(b, 12)[7]
    n_b = expected(b, 12).index(eos) + 1
    ra = sched.add(Request(a, max_tokens=30))
    rb = sched.add(Request(b, max_tokens=12, eos_ids=[eos]))          # ends early: a staged pass goes stale
    out = {ra: [], rb: []}
    late = None
    passes = 0
    while sched.has_work():
        passes += 1
        if passes == 15:
            late = sched.add(Request([8, 8], max_tokens=5))           # joins: another stale pass
            out[late] = []
        for ev in sched.step():
            assert ev.finish != "error"
            if ev.token is not None:
                out[ev.id].append(ev.token)
        eng.cache.check()
    assert out[ra] == expected(a, 30) and out[rb] == expected(b, 12)[:n_b] and out[late] == expected([8, 8], 5)
    assert eng.ran_staged > 10 and eng.discarded >= 2
    assert eng.staged == eng.ran_staged + eng.discarded or sched.staged is not None
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_passes_are_staged_while_a_waiting_request_has_no_slot_to_take():
    """With every slot taken a waiting request cannot join until one ends, so the running ones' next
    pass is staged all the same; when one ends the waiting request takes its slot and everybody's
    tokens are what they would have been."""
    rng = np.random.default_rng(11)
    ps = prompts(rng, [5, 9, 7, 12])
    lengths = [6, 14, 9, 8]
    eng = StagingEngine(pages=64, max_sequences=2)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=64, max_sequences=2))
    rids = [sched.add(Request(p, max_tokens=n)) for p, n in zip(ps, lengths)]
    staged_while_waiting = 0
    out = {}
    while sched.has_work():
        waiting_before, staged_before = len(sched.waiting), eng.ran_staged
        for ev in sched.step():
            if ev.token is not None:
                out.setdefault(ev.id, []).append(ev.token)
        if waiting_before and eng.ran_staged > staged_before:
            staged_while_waiting += 1
    assert staged_while_waiting >= 5, staged_while_waiting
    for rid, p, n in zip(rids, ps, lengths):
        assert out[rid] == expected(p, n)
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_portions_under_a_token_budget_decodes_first():
    eng = FakeEngine(pages=32)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=7, max_sequences=8))
    ps = prompts(np.random.default_rng(0), [20, 3, 9])
    ids = [sched.add(Request(p, max_tokens=5)) for p in ps]
    out, fin = run(sched)
    for rid, p in zip(ids, ps):
        assert out[rid] == expected(p, 5) and fin[rid][0] == "length"
    assert all(sum(c for _, c in p) <= 7 for p in eng.passes)
    assert eng.passes[0] == [(0, 7)] and eng.passes[1] == [(0, 7)] and eng.passes[2] == [(0, 6), (1, 1)]
    # once request 0 decodes, its single token comes before any portion of a prompt
    third = eng.passes[3]
    assert third[0] == (0, 1)
    assert eng.cache.free_pages() == eng.cache.total_pages()
    eng.cache.check()


def test_requests_arriving_in_the_middle():
    eng = FakeEngine(pages=32)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=16))
    rng = np.random.default_rng(1)
    ps = prompts(rng, [30, 5, 17, 2])
    out, ids = {}, []
    ids.append(sched.add(Request(ps[0], max_tokens=12)))
    for i in range(200):
        if i in (2, 5, 9):
            ids.append(sched.add(Request(ps[len(ids)], max_tokens=12)))
        for ev in sched.step():
            if ev.token is not None:
                out.setdefault(ev.id, []).append(ev.token)
        if not sched.has_work() and len(ids) == 4:
            break
    for rid, p in zip(ids, ps):
        assert out[rid] == expected(p, 12)


def test_eos_stop_and_ignore_eos():
    eng = FakeEngine(pages=32)
    sched = Scheduler(eng)
    p = [1, 2, 3]
    exp = expected(p, 8)
    a = sched.add(Request(p, max_tokens=8, eos_ids=[exp[2]]))
    b = sched.add(Request(p, max_tokens=8, eos_ids=[exp[2]], ignore_eos=True))
    c = sched.add(Request(p, max_tokens=8, stop=[exp[3:5]]))
    out, fin = run(sched)
    assert out[a] == exp[:3] and fin[a][0] == "eos"
    assert out[b] == exp and fin[b][0] == "length"
    assert out[c] == exp[:5] and fin[c][0] == "stop"


def test_pages_run_out_the_last_admitted_is_suspended_and_computed_again():
    """pages = the longest request's need + 3 (crates/kapel-infer/tests/engine.rs forces suspensions the
    same way): every request still gets the tokens it would get alone, and all pages end free."""
    rng = np.random.default_rng(2)
    ps = prompts(rng, [40, 33, 17, 25, 60])
    n_new = 30
    longest = -(-(60 + n_new + 1) // 16)
    eng = FakeEngine(pages=longest + 3)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=24))
    ids = [sched.add(Request(p, max_tokens=n_new)) for p in ps]
    out, fin = run(sched)
    for rid, p in zip(ids, ps):
        assert out[rid] == expected(p, n_new), f"request {rid}"
        assert fin[rid][0] == "length"
    st = sched.stats()
    assert st.preemptions > 0
    assert st.free_pages == st.pages and st.running == 0 and st.waiting == 0
    eng.cache.check()


def test_alone_and_still_too_long_ends_with_cache_full():
    eng = FakeEngine(pages=2)
    sched = Scheduler(eng)
    a = sched.add(Request(list(range(40)), max_tokens=4))        # 41 positions need 3 pages: never fits
    b = sched.add(Request([1, 2, 3], max_tokens=40))             # fits at first, outgrows 2 pages at 32 positions
    out, fin = run(sched)
    assert fin[a][0] == "error" and "cache full" in fin[a][1] and a not in out
    assert fin[b][0] == "error" and "cache full" in fin[b][1]
    assert out[b] == expected([1, 2, 3], len(out[b])) and len(out[b]) == 30
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_cancel_frees_pages_and_max_sequences_bounds_the_running():
    eng = FakeEngine(pages=32)
    sched = Scheduler(eng, EngineOptions(max_sequences=2))
    ids = [sched.add(Request([1, 2, 3, 4], max_tokens=50)) for _ in range(4)]
    sched.step()
    st = sched.stats()
    assert st.running == 2 and st.waiting == 2
    sched.cancel(ids[0])
    sched.cancel(ids[3])
    sched.step()
    assert sched.stats().running == 2 and sched.stats().waiting == 0
    for rid in ids:
        sched.cancel(rid)
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_a_failed_pass_ends_every_running_request():
    eng = FakeEngine(pages=32)
    sched = Scheduler(eng)
    ids = [sched.add(Request([1, 2, 3], max_tokens=5)) for _ in range(2)]
    sched.step()

    def boom(entries):
        raise RuntimeError("injected")

    eng.step = boom
    events = sched.step()
    assert sorted(e.id for e in events) == ids and all(e.finish == "error" and "injected" in e.error for e in events)
    assert not sched.has_work() and eng.cache.free_pages() == eng.cache.total_pages()


def test_windowed_group_counts_its_own_pages():
    """With a window the windowed group needs far fewer pages than the sequence is long."""
    eng = FakeEngine(pages=12, window=16)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=16))
    p = prompts(np.random.default_rng(3), [100])[0]
    rid = sched.add(Request(p, max_tokens=40))
    out, fin = run(sched)
    assert out[rid] == expected(p, 40)
    assert eng.cache.released_pages > 0


def test_temperature_uses_the_requests_own_seeded_sampler():
    eng = FakeEngine(pages=32)

    def flat(entries):                     # equal logits: the draw alone decides
        counts = [(e.id, len(e.tokens)) for e in entries]
        plan = eng.cache.plan(counts)
        eng.cache.commit(plan)
        return np.zeros((sum(len(e.want) for e in entries), VOCAB))

    eng.step = flat
    def tokens(seed):
        sched = Scheduler(eng)
        rid = sched.add(Request([1, 2], sampling=Sampling(temperature=0.8, seed=seed), max_tokens=20))
        return run(sched)[0][rid]

    a, b, c = tokens(7), tokens(7), tokens(8)
    assert a == b and a != c and len(set(a)) > 5


def test_a_reserve_keeps_a_share_of_the_pool_free_at_admission():
    """With `reserve`, a newcomer is admitted only if what the running requests will still take, its
    own need and ceil(reserve x pages) fit what is free (Kapel: engine.rs:355-388); alone, a request
    takes what there is."""
    rng = np.random.default_rng(11)
    ps = prompts(rng, [40, 40, 40])                       # each needs ceil((40 + 1) / 16) = 3 pages to start
    greedy = Sampling()

    eng = FakeEngine(pages=10)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=256, max_sequences=8, reserve=0.0))
    rids = [sched.add(Request(prompt=p, sampling=greedy, max_tokens=4)) for p in ps]
    sched.step()
    assert sched.stats().running == 3                      # 9 of 10 pages promised: all three fit

    eng = FakeEngine(pages=10)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=256, max_sequences=8, reserve=0.3))
    rids = [sched.add(Request(prompt=p, sampling=greedy, max_tokens=4)) for p in ps]
    first = sched.step()
    st = sched.stats()
    assert st.running == 2 and st.waiting == 1             # 3 + 3 + margin 3 <= 10, but 9 + 3 > 10
    out, finishes = run(sched)
    for ev in reversed(first):                              # the first pass's tokens come before the rest
        if ev.token is not None:
            out.setdefault(ev.id, []).insert(0, ev.token)
    for rid, p in zip(rids, ps):                            # the third ran once the others had ended
        assert out[rid] == expected(p, 4) and finishes[rid][0] == "length"
    assert sched.stats().free_pages == sched.stats().pages

    eng = FakeEngine(pages=4)                              # alone: the margin does not keep it out
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=256, max_sequences=8, reserve=0.9))
    rid = sched.add(Request(prompt=ps[0], sampling=greedy, max_tokens=3))
    out, finishes = run(sched)
    assert out[rid] == expected(ps[0], 3)


class LimitedEngine(FakeEngine):
    """The stand-in with a limit on positions, refusing what passes it as the step function does."""

    def __init__(self, limit, **kw):
        super().__init__(**kw)
        self.max_positions = limit

    def step(self, entries):
        for e in entries:
            if self.cache.length(e.id) + len(e.tokens) > self.max_positions:
                raise ValueError(f"request {e.id!r} would pass {self.max_positions} positions")
        return super().step(entries)


def test_a_request_that_reaches_the_position_limit_ends_alone_with_length():
    """One request reaches max_position_embeddings while another decodes beside it: the first ends
    with "length" after the last token it can be given, the second goes on and finishes normally,
    and the step function's own refusal is never met."""
    eng = LimitedEngine(40, pages=32)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=16))
    long_prompt, short_prompt = [3] * 30, [4, 5, 6]
    a = sched.add(Request(long_prompt, max_tokens=100))
    b = sched.add(Request(short_prompt, max_tokens=25))
    out, fin = run(sched)
    # positions 0..39 can be fed: the prompt's 30 and 10 generated tokens; the 11th token is the last given
    assert fin[a] == ("length", None) and out[a] == expected(long_prompt, 11)
    assert fin[b] == ("length", None) and out[b] == expected(short_prompt, 25)
    assert eng.cache.free_pages() == eng.cache.total_pages()
    with pytest.raises(ValueError, match="longer than the 40 positions"):
        sched.add(Request([1] * 41, max_tokens=1))
    c = sched.add(Request([1] * 40, max_tokens=5))          # exactly the limit: one token, then "length"
    out, fin = run(sched)
    assert out[c] == expected([1] * 40, 1) and fin[c][0] == "length"


def test_a_staged_pass_is_not_taken_beyond_the_position_limit():
    class Both(StagingEngine):
        max_positions = 24

    eng = Both(pages=32)
    sched = Scheduler(eng, EngineOptions(max_pass_tokens=16))
    a = sched.add(Request([2] * 10, max_tokens=100))
    out, fin = run(sched)
    assert out[a] == expected([2] * 10, 15) and fin[a][0] == "length"
    assert eng.cache.free_pages() == eng.cache.total_pages() and eng.ran_staged > 5


def test_two_schedulers_over_one_engine_never_share_a_request_id():
    """A stream that is not exhausted beside another call: both schedulers name sequences in the
    one cache, so their ids come from one counter, and ending one request leaves the other's pages."""
    eng = FakeEngine(pages=32)
    s1, s2 = Scheduler(eng), Scheduler(eng)
    p1, p2 = [1, 2, 3, 4], [9, 8, 7]
    a = s1.add(Request(p1, max_tokens=6))
    b = s2.add(Request(p2, max_tokens=6))
    assert a != b
    out = {a: [], b: []}
    for _ in range(3):                                       # both are live at once
        for s in (s1, s2):
            for ev in s.step():
                out[ev.id].append(ev.token)
    s1.cancel(a)                                             # one ends early; the other's pages stay
    eng.cache.check()
    while s2.has_work():
        for ev in s2.step():
            out[ev.id].append(ev.token)
    assert out[b] == expected(p2, 6) and out[a] == expected(p1, 3)
    assert eng.cache.free_pages() == eng.cache.total_pages()
