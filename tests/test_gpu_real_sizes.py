"""The engine at the real sizes of Gemma 2 against the plain implementation: the full vocabulary of
256,000, the window of 4,096 crossed by a request of 4,300 tokens, the real head counts and head
sizes; Gemma 2 2B at its full depth of 26 layers, 9B and 27B with as many of their layers as a
test's time allows (the test ids name both numbers). Each in 32-bit and in bfloat16, cut four
ways: whole; most of it in one step and the last 32 tokens one by one; in portions of changing
size; and beside a second request. Logits are compared at a handful of positions: the first, the
last before the window starts to move, the first after, the last, and the places where cuts fall.

The plain side is `plain_gemma2.forward_streamed` in 64-bit on the GPU (torch as an array library;
one layer's weights at a time). The model folder is written once per size, with values drawn on
the GPU, and both sides read it. Kapel checks the same things on whole models:
crates/kapel-models/tests/parity.rs:43-88,133-186 and crates/kapel-cuda/tests/parity.rs:53-113.
"""
import json
import shutil
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gemma2 as P
from helpers import ROOT, TOL, TraceBuilder, compare_trace, embed_scale_for, make_model_dir, random_tokens, run_trace_engine

pytestmark = pytest.mark.gpu

PRESETS = ROOT / "kapel_b200" / "config" / "presets"
# name -> (preset, layers built); the ids say "<built>-of-<the model's>"
SIZES = {"2b-26-of-26-layers": ("gemma2-2b", 26), "9b-6-of-42-layers": ("gemma2-9b", 6), "27b-4-of-46-layers": ("gemma2-27b", 4)}
LENGTH_A, LENGTH_B = 4300, 300
# bfloat16 bounds at about twice what each size shows (1.0e-2 through 26 layers, 2.6e-3 through 6 and 4)
TOL_BF16_DEEP = {"2b-26-of-26-layers": 2e-2, "9b-6-of-42-layers": 6e-3, "27b-4-of-46-layers": 6e-3}


def _traces(a, b):
    """The four cuts as traces over requests `a` (crosses the window) and `b`."""
    n = len(a)
    whole = TraceBuilder()
    whole.step([("a", a, [0, 4094, 4095, 4096, 4097, n - 1])], end=["a"])
    whole.step([("b", b, [0, len(b) - 1])], end=["b"])

    last32 = TraceBuilder()
    head = n - 32
    last32.step([("a", a[:head], [head - 1])])
    for i in range(head, n):
        last32.step([("a", [a[i]], [0])], end=["a"] if i == n - 1 else [])

    portions = TraceBuilder()
    at = 0
    for size in (1500, 2, 1000, 594, 1000, 7, n - 4103):        # a portion ends at 4,095 and the next starts at 4,096
        portions.step([("a", a[at : at + size], [0, size - 1] if size > 1 else [0])], end=["a"] if at + size == n else [])
        at += size
    assert at == n

    mixed = TraceBuilder()
    mixed.step([("a", a[:2000], [1999]), ("b", b[:2], [1])])
    mixed.step([("a", a[2000:4090], [2089]), ("b", b[2:250], [247])])
    mixed.step([("a", a[4090:4100], list(range(10))), ("b", [b[250]], [0])])      # a's rows straddle the window's first move
    for i in range(8):                                                           # both decode
        mixed.step([("a", [a[4100 + i]], [0]), ("b", [b[251 + i]], [0])])
    mixed.step([("a", a[4108:], [n - 4109]), ("b", b[259:], [len(b) - 260])], end=["a", "b"])
    return {"whole": whole, "last 32 one by one": last32, "portions": portions, "mixed": mixed}


@pytest.fixture(scope="module", params=list(SIZES))
def case(request):
    name = request.param
    preset, layers = SIZES[name]
    raw = dict(json.loads((PRESETS / f"{preset}.json").read_text()), num_hidden_layers=layers)
    folder = make_model_dir(raw, seed=17, device="cuda")
    rng = np.random.default_rng(51)
    a, b = random_tokens(rng, LENGTH_A, raw["vocab_size"]), random_tokens(rng, LENGTH_B, raw["vocab_size"])
    traces = _traces(a, b)
    wanted = {"a": set(), "b": set()}
    for tb in traces.values():
        for rows in tb.rows.values():
            for rid, pos in rows:
                wanted[rid].add(pos)
    order = {rid: sorted(s) for rid, s in wanted.items()}
    plain = {}
    for dtype in ("float32", "bfloat16"):
        scale = embed_scale_for(raw, dtype)
        key = round(scale, 6)
        if key not in plain:
            out = P.forward_streamed(folder, [(a, order["a"], scale), (b, order["b"], scale)], torch.float64, "cuda")
            plain[key] = {rid: {pos: out[i][j].numpy() for j, pos in enumerate(order[rid])} for i, rid in enumerate(("a", "b"))}
        plain[dtype] = plain[key]
    torch.cuda.empty_cache()
    yield name, raw, folder, traces, plain
    shutil.rmtree(folder, ignore_errors=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_sizes_in_four_cuts(case, dtype):
    from kapel_b200.engine import Engine

    name, raw, folder, traces, plain = case
    tol = TOL["float32"] if dtype == "float32" else TOL_BF16_DEEP[name]
    engine = Engine.from_dir(folder, dtype=dtype, max_tokens=LENGTH_A + LENGTH_B + 256, max_sequences=4)
    assert not engine.unexpected_tensors
    for cut, tb in traces.items():
        got = run_trace_engine(engine, tb.steps)
        worst = compare_trace(got, tb, plain[dtype], tol, f"{name} {cut} {dtype}")
        print(f"{name} {dtype} {cut}: worst {worst:.2e}")
        engine.cache.check()
        assert engine.cache.free_pages() == engine.cache.total_pages()
    assert engine.cache.released_pages > 0                # the window passed pages of the long request
    engine.check()
