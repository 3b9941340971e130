"""Generation through the entry points, the replay program, long decoding, first tokens,
and the scheduler over the real engine with so few pages that requests are suspended."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_gemma2 as P
from helpers import (ROOT, TINY, TOL, TraceBuilder, compare_trace, embed_scale_for, make_model_dir, plain_logits,
                     plain_model, random_tokens, run_trace_engine, run_trace_program)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders():
    return {name: make_model_dir(raw, seed) for name, (raw, seed) in TINY.items()}


def plain_greedy(folder, raw, prompt, n, dtype="float32"):
    cfg, w = plain_model(folder)
    seq = list(prompt)
    margins = []
    for _ in range(n):
        row = P.forward(cfg, w, seq, embed_scale=embed_scale_for(raw, dtype))[-1].numpy()
        order = np.argsort(row)
        margins.append(float(row[order[-1]] - row[order[-2]]))
        seq.append(int(order[-1]))
    return seq[len(prompt):], margins


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """Tiny A: prompts of 5, 17, 33, 40 and 24 greedy tokens each; in 32-bit the tokens are the plain ones."""
    import kapel_b200

    raw, _ = TINY[name]
    rng = np.random.default_rng(21)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in ([5, 17, 33, 40] if name == "A" else [1, 50, 90])]
    model = kapel_b200.Model(str(folders[name]), device="cuda", dtype="f32", max_tokens_cached=512, max_sequences=8)
    want = [plain_greedy(folders[name], raw, p, 24) for p in prompts]
    for p, (tokens, margins) in zip(prompts, want):
        got = model.generate(p, max_tokens=24)
        assert got == tokens, f"prompt of {len(p)}: {got} != {tokens} (smallest margin {min(margins):.2e})"
        assert list(model.generate(p, max_tokens=24, stream=True)) == tokens
    assert model.generate_batch(prompts, max_tokens=24) == [t for t, _ in want], "together = each alone"
    assert model.engine.recorded_passes > 0, "decode steps went through recordings"
    # bfloat16: the same tokens as long as the plain margin is well above bfloat16's error
    bf = kapel_b200.Model(str(folders[name]), device="cuda", dtype="bf16", max_tokens_cached=512, max_sequences=8)
    for p, (tokens, margins) in zip(prompts, want):
        got = bf.generate(p, max_tokens=24)
        safe = next((i for i, m in enumerate(margins) if m < 0.05), len(margins))
        assert got[:safe] == tokens[:safe]
    assert model.engine.cache.free_pages() == model.engine.cache.total_pages()


def test_temperature_same_seed_same_tokens_and_chunked_prefill(folders):
    """Tiny B's workload: prompts 1, 50, 90 in portions of 32 mixed with decodes, 40 steps at 0.8, seed 7."""
    import kapel_b200

    raw, _ = TINY["B"]
    rng = np.random.default_rng(22)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in (1, 50, 90)]
    model = kapel_b200.Model(str(folders["B"]), dtype="f32", max_tokens_cached=512, max_sequences=8)
    a = model.generate_batch(prompts, max_tokens=40, temperature=0.8, seed=7, max_pass_tokens=32)
    b = model.generate_batch(prompts, max_tokens=40, temperature=0.8, seed=7, max_pass_tokens=32)
    c = model.generate_batch(prompts, max_tokens=40, temperature=0.8, seed=8, max_pass_tokens=32)
    assert a == b and a != c and all(len(x) == 40 for x in a)
    # request i draws with seed + i: alone with that seed it gets the same tokens
    assert model.generate(prompts[1], max_tokens=40, temperature=0.8, seed=8) == a[1]
    # the filters run on the host with the same generator
    d = model.generate(prompts[2], max_tokens=10, temperature=0.8, top_k=5, top_p=0.9, seed=3)
    assert d == model.generate(prompts[2], max_tokens=10, temperature=0.8, top_k=5, top_p=0.9, seed=3)
    assert model.generate(prompts[2], max_tokens=5, temperature=0.8, top_k=1, seed=3) == model.generate(prompts[2], max_tokens=5)


@pytest.mark.parametrize("route", ["device", "host"])
def test_sampled_tokens_are_the_plain_samplers_over_the_plain_logits(folders, route):
    """Tiny B's workload in 32-bit: prompts of 1, 50 and 90 in portions of 32 beside decoded tokens,
    40 tokens each at temperature 0.8 with seed 7 (request i draws with seed 7 + i). Every token the
    engine gives is the one the plain sampler draws, with the same uniform number, from the plain
    logits of the sequence so far; a difference is allowed only where the plain running total of
    probabilities passes the uniform number by less than 1e-5. `device`: the draw is made where the
    logits are (32-bit softmax); `host`: a min_p too small to remove anything sends it through the
    host sampler (64-bit)."""
    import kapel_b200

    raw, _ = TINY["B"]
    rng = np.random.default_rng(22)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in (1, 50, 90)]
    model = kapel_b200.Model(str(folders["B"]), dtype="f32", max_tokens_cached=512, max_sequences=8)
    extra = {} if route == "device" else {"min_p": 1e-30}
    got = model.generate_batch(prompts, max_tokens=40, temperature=0.8, seed=7, max_pass_tokens=32, **extra)
    near = 0
    for i, (prompt, tokens) in enumerate(zip(prompts, got)):
        assert len(tokens) == 40
        logits = plain_logits(folders["B"], prompt + tokens, embed_scale=embed_scale_for(raw, "float32"))
        draws = P.PlainRng(7 + i)
        for t, token in enumerate(tokens):
            u = draws.uniform()
            row = [float(x) for x in logits[len(prompt) - 1 + t]]
            want = P.plain_choose(row, 0.8, u)
            if token != want:
                scaled = np.asarray(row) / 0.8
                prob = np.exp(scaled - scaled.max())
                running = np.cumsum(prob / prob.sum())
                lo, hi = min(token, want), max(token, want)
                assert hi == lo + 1 and abs(running[lo] - u) < 1e-5, \
                    f"request {i}, token {t}: engine {token}, plain {want}, u {u}, running total {running[lo]}"
                near += 1
    assert near <= 2, f"{near} draws fell on a boundary: too many for chance"


def test_scheduler_with_few_pages_suspends_and_still_gives_each_its_tokens(folders):
    import kapel_b200
    from kapel_b200.engine.scheduler import Request

    raw, _ = TINY["A"]
    rng = np.random.default_rng(23)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in (40, 33, 17, 5, 28)]
    n_new = 20
    alone = kapel_b200.Model(str(folders["A"]), dtype="f32", max_tokens_cached=256, max_sequences=2)
    want = [alone.generate(p, max_tokens=n_new) for p in prompts]
    pages = -(-(40 + n_new + 1) // 16) + 3
    small = kapel_b200.Model(str(folders["A"]), dtype="f32", max_tokens_cached=pages * 16, max_sequences=8)
    sched = small.scheduler(max_pass_tokens=24)
    ids = [sched.add(Request(p, max_tokens=n_new)) for p in prompts]
    out = {r: [] for r in ids}
    while sched.has_work():
        for ev in sched.step():
            assert ev.finish != "error", ev.error
            if ev.token is not None:
                out[ev.id].append(ev.token)
    assert [out[r] for r in ids] == want
    st = sched.stats()
    assert st.preemptions > 0 and st.free_pages == st.pages
    small.engine.cache.check()


def test_passes_staged_ahead_give_the_same_tokens_and_hold_no_page_afterwards(folders):
    """While a decode pass runs the scheduler stages the next one (pages taken, inputs written,
    only the token ids open). The tokens are those of each request alone; a request that meets
    its end-of-sequence token, one that is cancelled and one that joins late all make a staged
    pass stale, which must give its pages back."""
    import kapel_b200
    from kapel_b200.engine.scheduler import Request

    raw, _ = TINY["A"]
    rng = np.random.default_rng(29)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in (20, 31, 9, 14)]
    model = kapel_b200.Model(str(folders["A"]), dtype="f32", max_tokens_cached=1024, max_sequences=8)
    want = [model.generate(p, max_tokens=40) for p in prompts]
    eos = want[1][17]                                   # request 1 stops where this token first appears
    cut = want[1].index(eos) + 1
    sched = model.scheduler(max_pass_tokens=64)
    ids = [sched.add(Request(prompts[0], max_tokens=40)), sched.add(Request(prompts[1], max_tokens=40, eos_ids=[eos])),
           sched.add(Request(prompts[2], max_tokens=40))]
    out = {r: [] for r in ids}
    passes = 0
    while sched.has_work():
        passes += 1
        if passes == 12:                                # a request joins while others decode
            ids.append(sched.add(Request(prompts[3], max_tokens=40)))
            out[ids[-1]] = []
        if passes == 25:
            sched.cancel(ids[2])
        for ev in sched.step():
            assert ev.finish != "error", ev.error
            if ev.token is not None:
                out[ev.id].append(ev.token)
        model.engine.cache.check()
    assert out[ids[0]] == want[0]
    assert out[ids[1]] == want[1][:cut]
    assert out[ids[2]] == want[2][: len(out[ids[2]])] and 0 < len(out[ids[2]]) < 40
    assert out[ids[3]] == want[3]
    assert sched.staged_passes > 10, "decode passes ran from staged plans"
    assert sched.staged is None or not model.engine.cache._sequences
    assert model.engine.cache.free_pages() == model.engine.cache.total_pages()


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_passes_enqueued_ahead_of_the_host_give_the_same_tokens(folders, temperature):
    """Where the tokens are chosen on the device, the pass after is fed them from device memory and
    enqueued before the host has read them. The tokens are those of a scheduler that waits for every
    token first; a request that meets its end-of-sequence token while the pass after it is already
    on its way ends there (the row that pass computed for it is dropped), one that is cancelled and
    one that joins late change the running set in mid-flight, and no page is lost."""
    import kapel_b200
    from kapel_b200.engine.scheduler import Request
    from kapel_b200.sampling import Sampling

    raw, _ = TINY["B"]
    rng = np.random.default_rng(31)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in (20, 31, 9, 14)]
    model = kapel_b200.Model(str(folders["B"]), dtype="f32", max_tokens_cached=1024, max_sequences=8)

    def run(run_ahead, eos):
        sched = model.scheduler(max_pass_tokens=64, run_ahead=run_ahead)
        def request(i, **kw):
            return Request(prompts[i], sampling=Sampling(temperature=temperature, seed=5 + i), max_tokens=40, **kw)
        ids = [sched.add(request(0)), sched.add(request(1, eos_ids=eos)), sched.add(request(2))]
        out = {r: [] for r in ids}
        passes = 0
        while sched.has_work():
            passes += 1
            if passes == 12:
                ids.append(sched.add(request(3)))
                out[ids[-1]] = []
            if passes == 25:
                sched.cancel(ids[2])
            for ev in sched.step():
                assert ev.finish != "error", ev.error
                if ev.token is not None:
                    out[ev.id].append(ev.token)
            model.engine.cache.check()
        assert model.engine.cache.free_pages() == model.engine.cache.total_pages()
        return [out[r] for r in ids], sched

    plain, waited = run(False, [])
    assert waited.ahead_passes == 0 and waited.staged_passes > 10
    eos = [plain[1][17]]
    want, _ = run(False, eos)
    got, sched = run(True, eos)
    assert got == want
    assert len(got[1]) == want[1].index(eos[0]) + 1 < 40 and len(got[0]) == 40 and len(got[3]) == 40 and 0 < len(got[2]) < 40
    assert sched.ahead_passes > 10, "decode passes were enqueued ahead of the host"


def test_settle_reads_the_pass_on_its_way_and_leaves_the_cache_one_token_behind(folders):
    """After passes enqueued ahead of the host, `settle` gives the tokens of the pass on its way and
    frees what was staged: every request's cache then holds all its tokens but the last, and stepping
    the engine directly from there continues the sequence as the scheduler would have."""
    import kapel_b200
    from kapel_b200.engine import StepEntry
    from kapel_b200.engine.scheduler import Request
    from kapel_b200.sampling import Sampling

    raw, _ = TINY["A"]
    rng = np.random.default_rng(41)
    prompts = [random_tokens(rng, n, raw["vocab_size"]) for n in (12, 27)]
    model = kapel_b200.Model(str(folders["A"]), dtype="f32", max_tokens_cached=512, max_sequences=4)

    def tokens_of(run_ahead, n):
        sched = model.scheduler(max_pass_tokens=64, run_ahead=run_ahead)
        ids = [sched.add(Request(p, sampling=Sampling(), max_tokens=60, ignore_eos=True)) for p in prompts]
        for _ in range(n):
            sched.step()
        return sched, ids

    want_sched, want_ids = tokens_of(False, 30)
    want = [list(want_sched.entries[r].sequence) for r in want_ids]
    for r in want_ids:
        want_sched.cancel(r)
    sched, ids = tokens_of(True, 14)
    assert sched.ahead is not None and sched.ahead_passes > 5, "a pass is on its way"
    given = sched.settle()
    assert len(given) == 2 and sched.ahead is None and sched.staged is None
    engine = model.engine
    seqs = {r: list(sched.entries[r].sequence) for r in ids}
    for r in ids:
        assert engine.cache.length(r) == len(seqs[r]) - 1
    while len(seqs[ids[0]]) < len(want[0]):
        logits = engine.step([StepEntry(r, [seqs[r][-1]], [0]) for r in ids])
        for r, row in zip(ids, logits.argmax(dim=-1).tolist()):
            seqs[r].append(int(row))
    assert [seqs[r] for r in ids] == want
    for r in ids:
        sched.cancel(r)
    engine.cache.check()
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folders, dtype):
    """A one-token prompt, then every token one by one up to the model's limit: first tokens of a
    sequence, page edges, the window passing pages, recordings replayed throughout."""
    from kapel_b200.engine import Engine

    for name in ("A", "B"):
        raw, _ = TINY[name]
        n = raw["max_position_embeddings"]
        toks = random_tokens(np.random.default_rng(24), n, raw["vocab_size"])
        plain = {"s": plain_logits(folders[name], toks, embed_scale=embed_scale_for(raw, dtype))}
        engine = Engine.from_dir(folders[name], dtype=dtype, max_tokens=n, max_sequences=2)
        tb = TraceBuilder()
        for i, t in enumerate(toks):
            tb.step([("s", [t], [0])], end=["s"] if i == n - 1 else [])
        worst = compare_trace(run_trace_engine(engine, tb.steps), tb, plain, TOL[dtype], f"long {name} {dtype}")
        print(f"long decode {name} {dtype}: {n} tokens, worst {worst:.2e}")
        assert engine.recorded_passes == n
        with pytest.raises(ValueError, match="allows"):
            engine.step([("t", toks + [1], [0])])
        assert engine.cache.free_pages() == engine.cache.total_pages()


def test_recorded_step_equals_eager_step_bit_for_bit(folders):
    from kapel_b200.engine import Engine

    raw, _ = TINY["B"]
    toks = random_tokens(np.random.default_rng(25), 60, raw["vocab_size"])
    outs = []
    for graphs in (True, False):
        engine = Engine.from_dir(folders["B"], dtype="bfloat16", max_tokens=128, max_sequences=4, graphs=graphs)
        tb = TraceBuilder()
        tb.step([("a", toks[:30], [29]), ("b", toks[:7], [6])])
        for i in range(30, 60):
            tb.step([("a", [toks[i]], [0]), ("b", [toks[i - 23]], [0])])
        res = run_trace_engine(engine, tb.steps)
        outs.append(np.concatenate([res[s] for s in sorted(res)]))
        assert (engine.recorded_passes > 0) == graphs
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recorded_prompt_passes_equal_eager_ones_bit_for_bit(folders, dtype):
    """Prompts of one length cut into portions of 80 tokens repeat their passes' shapes (80 behind 0,
    behind 80, 70 behind 160): the second request's passes are recorded, the later ones replayed, on
    other tokens and, since requests end in between, on other pages. Every logit is what an engine
    without recordings gives, bit for bit; a recording that fails to be made loses only itself."""
    from kapel_b200.engine import Engine

    raw, _ = TINY["B"]
    rng = np.random.default_rng(52)
    prompts = [random_tokens(rng, 230, raw["vocab_size"]) for _ in range(5)]
    outs = []
    for graphs in (True, False):
        engine = Engine.from_dir(folders["B"], dtype=dtype, max_tokens=512, max_sequences=4, graphs=graphs)
        if graphs:
            engine.prompt_graphs.fail_next_captures = 1          # the first recording fails: that pass runs eagerly, the shape is tried again later
        tb = TraceBuilder()
        for i, toks in enumerate(prompts):
            name = f"r{i}"
            tb.step([(name, toks[:80], [79])])
            tb.step([(name, toks[80:160], [0, 79])])
            tb.step([(name, toks[160:230], [69])], end=[name] if i % 2 == 0 else [])
            if i % 2 == 1:
                tb.step([(name, [toks[0]], [0])], end=[name])
        res = run_trace_engine(engine, tb.steps)
        outs.append(np.concatenate([res[s] for s in sorted(res)]))
        if graphs:
            pg = engine.prompt_graphs
            assert pg.failed_captures == 1 and len(pg.recorded) == 2 and pg.replays >= 8, (pg.failed_captures, len(pg.recorded), pg.replays)
        engine.cache.check()
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_any_length_share_recordings_of_round_lengths(folders, dtype):
    """A prompt alone in its pass is rounded up to a round number of rows, so that prompts of 66 to 96
    tokens are one shape: the third such prompt is replayed from the recording the second made. The
    rows added write nothing into the cache and are seen by nobody: every request's logits at its last
    prompt token and over the tokens decoded after it are the plain implementation's, and the pages
    are all given back."""
    from kapel_b200.engine import Engine, StepEntry

    raw, _ = TINY["B"]                                     # 256 positions
    rng = np.random.default_rng(61)
    lengths = [70, 96, 67, 91, 130, 150, 131]
    engine = Engine.from_dir(folders["B"], dtype=dtype, max_tokens=1024, max_sequences=4)
    for i, n in enumerate(lengths):
        toks = random_tokens(rng, n + 6, raw["vocab_size"])
        want = plain_logits(folders["B"], toks, embed_scale_for(raw, dtype))
        name = f"q{i}"
        got = [engine.step([StepEntry(name, toks[:n], [n - 1])]).float().cpu().numpy()[0]]
        for t in range(n, n + 6):
            got.append(engine.step([StepEntry(name, [toks[t]], [0])]).float().cpu().numpy()[0])
        for j, row in enumerate(got):
            ref = want[n - 1 + j]
            assert np.abs(row - ref).max() / np.abs(ref).max() < TOL[dtype], (n, j)
        engine.end(name)
        engine.cache.check()
    pg = engine.prompt_graphs
    assert len(pg.recorded) == 2 and pg.replays == 5, (len(pg.recorded), pg.replays)      # 96 rows: 4 prompts, 3 replays; 160 rows: 3 prompts, 2 replays
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, dtype):
    """bin/trace_run as a program: whole, then portions beside decoded tokens, pages used again."""
    raw, _ = TINY["A"]
    rng = np.random.default_rng(26)
    reqs = {f"r{i}": random_tokens(rng, n, raw["vocab_size"]) for i, n in enumerate([40, 17, 33, 64, 50])}
    plain = {r: plain_logits(folders["A"], t, embed_scale=embed_scale_for(raw, dtype)) for r, t in reqs.items()}
    tb = TraceBuilder()
    tb.step([("r0", reqs["r0"], range(40))], end=["r0"])
    tb.step([("r1", reqs["r1"][:9], [8]), ("r2", reqs["r2"][:2], [0, 1])])
    tb.step([("r1", reqs["r1"][9:10], [0]), ("r2", reqs["r2"][2:20], [17]), ("r3", reqs["r3"][:33], [])])
    tb.step([("r3", reqs["r3"][33:], [30])])                     # r1 and r2 are left out of this step
    tb.step([("r1", reqs["r1"][10:], [6]), ("r2", reqs["r2"][20:], [12])], end=["r1", "r2", "r3"])
    tb.step([("r4", reqs["r4"], [0, 49])], end=["r4"])
    res = run_trace_program(folders["A"], dtype, tb.steps, max_tokens=192)
    compare_trace(res, tb, plain, TOL[dtype], f"program {dtype}")
    assert 3 in res and res[3].shape == (1, raw["vocab_size"])


def test_command_line(folders):
    raw, _ = TINY["A"]
    prompt = random_tokens(np.random.default_rng(27), 12, raw["vocab_size"])
    want, _ = plain_greedy(folders["A"], raw, prompt, 8)
    cmd = [sys.executable, "-m", "kapel_b200", "run", str(folders["A"]), "--tokens", ",".join(map(str, prompt)),
           "--max-tokens", "8", "--greedy", "--dtype", "f32", "--stats"]
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=str(ROOT), timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.strip().splitlines()[-1].split(",")] == want
    assert "tokens/s" in r.stderr
    r = subprocess.run(cmd[:5] + ["--quantize", "int8", "--tokens", "1"], capture_output=True, text=True, cwd=str(ROOT), timeout=600)
    assert r.returncode == 1 and "quantized" in r.stderr


def test_command_line_with_random_weights_and_engine_options(folders, tmp_path):
    """`run --random CONFIG --seed-weights S --prompt-len N --pages --max-pass-tokens --max-sequences`:
    no folder, weights made on the device; the same tokens as the Python entry point gives for the
    same configuration, seeds and prompt; the prompt runs in portions of --max-pass-tokens."""
    import kapel_b200

    raw, _ = TINY["B"]
    config = tmp_path / "config.json"
    config.write_text(json.dumps(raw))
    cmd = [sys.executable, "-m", "kapel_b200", "run", "--random", str(config), "--seed-weights", "3", "--prompt-len", "21", "--seed", "5",
           "--pages", "6", "--max-pass-tokens", "8", "--max-sequences", "2", "--max-tokens", "6", "--greedy", "--dtype", "f32", "--stats"]
    r = subprocess.run(cmd, capture_output=True, text=True, cwd=str(ROOT), timeout=600)
    assert r.returncode == 0, r.stderr
    got = [int(t) for t in r.stdout.strip().splitlines()[-1].split(",")]
    prompt = [int(t) for t in np.random.default_rng(5).integers(0, raw["vocab_size"], size=21)]
    model = kapel_b200.Model.random(str(config), seed=3, dtype="f32", pages=6, max_sequences=2, max_pass_tokens=8)
    assert model.engine.cache.total_pages() == [6, 6]
    assert got == model.generate(prompt, max_tokens=6)
    assert "prompt 21 tokens" in r.stderr and "passes 8 " in r.stderr          # 3 portions of at most 8, then 5 more tokens
    r = subprocess.run(cmd[:4] + ["--tokens", "1"], capture_output=True, text=True, cwd=str(ROOT), timeout=600)
    assert r.returncode == 2 and "either MODEL or --random" in r.stderr
    r = subprocess.run([sys.executable, "-m", "kapel_b200", "run", "--random", "no-such-size", "--tokens", "1"],
                       capture_output=True, text=True, cwd=str(ROOT), timeout=600)
    assert r.returncode == 1 and "presets" in r.stderr
